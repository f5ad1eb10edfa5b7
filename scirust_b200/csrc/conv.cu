// Convolutional-network kernels on NHWC bf16 activations: im2col / col2im around the tcgen05 GEMM
// (explicit-GEMM convolution forward, input gradient and weight gradient), max pooling
// forward/backward, BatchNorm2d forward/backward with running statistics, ReLU and bias helpers.
//
// Reference semantics: im2col + GEMM convolution and its adjoints
// (scirust-core/src/nn/conv2d.rs:13-208, nn/conv_utils.rs:19-120; shader IM2COL / COL2IM
// scirust-gpu/src/conv_gpu.rs:7-120 with CPU oracles :122,172), max_pool2d
// (scirust-core/src/autodiff/reverse.rs:5038), BatchNorm2d with momentum 0.1, eps 1e-5 and an
// unbiased running variance (nn/batch_norm_2d.rs:18-90,177-190).
// Layout differs from the reference on purpose: activations are [B*H*W, C] (channels innermost) so
// that a convolution's output is directly the GEMM's row-major result and per-channel statistics
// are column reductions. Patch columns are ordered (kh, kw, c) and padded to a multiple of 8.
// All reductions (col2im, column statistics) use a fixed order; no atomics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "api.h"

namespace sb {

// col[(b,oh,ow), (kh,kw,c)] = x[b, oh*s - pad + kh, ow*s - pad + kw, c] (0 outside); Kp = padded width
__global__ void im2col_nhwc_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col, int B,
                                   int H, int W, int C, int KH, int KW, int stride, int pad, int OH, int OW,
                                   int Kp) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(B) * OH * OW * Kp;
  if (idx >= total) return;
  const int k = static_cast<int>(idx % Kp);
  const size_t row = idx / Kp;
  const int ow = static_cast<int>(row % OW);
  const int oh = static_cast<int>((row / OW) % OH);
  const int b = static_cast<int>(row / (static_cast<size_t>(OW) * OH));
  __nv_bfloat16 v = __float2bfloat16(0.f);
  if (k < KH * KW * C) {
    const int c = k % C;
    const int kw = (k / C) % KW;
    const int kh = k / (C * KW);
    const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
    if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = x[((static_cast<size_t>(b) * H + ih) * W + iw) * C + c];
  }
  col[idx] = v;
}

// The same gather, eight channels (16 bytes) per thread, for C a multiple of 8 (every layer but an RGB stem): one
// index decomposition per 16-byte word instead of per element, and 16-byte loads and stores.
__global__ void im2col_nhwc_vec8_kernel(const uint4* __restrict__ x, uint4* __restrict__ col, int B, int H, int W,
                                        int C8, int KH, int KW, int stride, int pad, int OH, int OW, int Kp8) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(B) * OH * OW * Kp8;
  if (idx >= total) return;
  const int k8 = static_cast<int>(idx % Kp8);
  const size_t row = idx / Kp8;
  const int ow = static_cast<int>(row % OW);
  const int oh = static_cast<int>((row / OW) % OH);
  const int b = static_cast<int>(row / (static_cast<size_t>(OW) * OH));
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (k8 < KH * KW * C8) {
    const int c8 = k8 % C8;
    const int kw = (k8 / C8) % KW;
    const int kh = k8 / (C8 * KW);
    const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
    if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = __ldg(x + ((static_cast<size_t>(b) * H + ih) * W + iw) * C8 + c8);
  }
  col[idx] = v;
}

__device__ __forceinline__ float conv_bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float conv_bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t conv_pack(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// col2im, eight channels per thread; the taps are added in the same ascending (kh, kw) order as the scalar kernel
__global__ void col2im_nhwc_vec8_kernel(const uint4* __restrict__ dcol, uint4* __restrict__ dx, int B, int H, int W,
                                        int C8, int KH, int KW, int stride, int pad, int OH, int OW, int Kp8) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(B) * H * W * C8;
  if (idx >= total) return;
  const int c8 = static_cast<int>(idx % C8);
  const int iw = static_cast<int>((idx / C8) % W);
  const int ih = static_cast<int>((idx / (static_cast<size_t>(C8) * W)) % H);
  const int b = static_cast<int>(idx / (static_cast<size_t>(C8) * W * H));
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int kh = 0; kh < KH; ++kh) {
    const int th = ih + pad - kh;
    if (th < 0 || th % stride) continue;
    const int oh = th / stride;
    if (oh >= OH) continue;
    for (int kw = 0; kw < KW; ++kw) {
      const int tw = iw + pad - kw;
      if (tw < 0 || tw % stride) continue;
      const int ow = tw / stride;
      if (ow >= OW) continue;
      const uint4 v = __ldg(dcol + ((static_cast<size_t>(b) * OH + oh) * OW + ow) * Kp8 + (kh * KW + kw) * C8 + c8);
      acc[0] += conv_bf_lo(v.x); acc[1] += conv_bf_hi(v.x); acc[2] += conv_bf_lo(v.y); acc[3] += conv_bf_hi(v.y);
      acc[4] += conv_bf_lo(v.z); acc[5] += conv_bf_hi(v.z); acc[6] += conv_bf_lo(v.w); acc[7] += conv_bf_hi(v.w);
    }
  }
  dx[idx] = make_uint4(conv_pack(acc[0], acc[1]), conv_pack(acc[2], acc[3]), conv_pack(acc[4], acc[5]),
                       conv_pack(acc[6], acc[7]));
}

// dx[b,ih,iw,c] = sum over (kh,kw) in ascending order of dcol[(b,oh,ow),(kh,kw,c)] where the output
// position maps onto this input pixel. Gather form: one thread per input element.
__global__ void col2im_nhwc_kernel(const __nv_bfloat16* __restrict__ dcol, __nv_bfloat16* __restrict__ dx, int B,
                                   int H, int W, int C, int KH, int KW, int stride, int pad, int OH, int OW,
                                   int Kp) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(B) * H * W * C;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % C);
  const int iw = static_cast<int>((idx / C) % W);
  const int ih = static_cast<int>((idx / (static_cast<size_t>(C) * W)) % H);
  const int b = static_cast<int>(idx / (static_cast<size_t>(C) * W * H));
  float acc = 0.f;
  for (int kh = 0; kh < KH; ++kh) {
    const int th = ih + pad - kh;
    if (th < 0 || th % stride) continue;
    const int oh = th / stride;
    if (oh >= OH) continue;
    for (int kw = 0; kw < KW; ++kw) {
      const int tw = iw + pad - kw;
      if (tw < 0 || tw % stride) continue;
      const int ow = tw / stride;
      if (ow >= OW) continue;
      acc += __bfloat162float(dcol[((static_cast<size_t>(b) * OH + oh) * OW + ow) * Kp + (kh * KW + kw) * C + c]);
    }
  }
  dx[idx] = __float2bfloat16_rn(acc);
}

// y = max over the k x k window; idx = flat offset (kh*k+kw) of the first maximum (for backward)
__global__ void maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                   uint8_t* __restrict__ arg, int B, int H, int W, int C, int k, int stride, int OH,
                                   int OW) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(B) * OH * OW * C;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % C);
  const int ow = static_cast<int>((idx / C) % OW);
  const int oh = static_cast<int>((idx / (static_cast<size_t>(C) * OW)) % OH);
  const int b = static_cast<int>(idx / (static_cast<size_t>(C) * OW * OH));
  float best = -INFINITY;
  int bi = 0;
  for (int kh = 0; kh < k; ++kh)
    for (int kw = 0; kw < k; ++kw) {
      const int ih = oh * stride + kh, iw = ow * stride + kw;
      if (ih < H && iw < W) {
        const float v = __bfloat162float(x[((static_cast<size_t>(b) * H + ih) * W + iw) * C + c]);
        if (v > best) { best = v; bi = kh * k + kw; }
      }
    }
  y[idx] = __float2bfloat16_rn(best);
  if (arg) arg[idx] = static_cast<uint8_t>(bi);
}
// windows may overlap (stride < k): gather form over input pixels, fixed (kh, kw) order
__global__ void maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const uint8_t* __restrict__ arg,
                                   __nv_bfloat16* __restrict__ dx, int B, int H, int W, int C, int k, int stride,
                                   int OH, int OW) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(B) * H * W * C;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % C);
  const int iw = static_cast<int>((idx / C) % W);
  const int ih = static_cast<int>((idx / (static_cast<size_t>(C) * W)) % H);
  const int b = static_cast<int>(idx / (static_cast<size_t>(C) * W * H));
  float acc = 0.f;
  for (int kh = 0; kh < k; ++kh) {
    const int th = ih - kh;
    if (th < 0 || th % stride) continue;
    const int oh = th / stride;
    if (oh >= OH) continue;
    for (int kw = 0; kw < k; ++kw) {
      const int tw = iw - kw;
      if (tw < 0 || tw % stride) continue;
      const int ow = tw / stride;
      if (ow >= OW) continue;
      const size_t o = ((static_cast<size_t>(b) * OH + oh) * OW + ow) * C + c;
      if (arg[o] == kh * k + kw) acc += __bfloat162float(dy[o]);
    }
  }
  dx[idx] = __float2bfloat16_rn(acc);
}

// Column statistics of a [rows, C] matrix in two fixed-order stages.
// stage 1: partial[chunk][0][c] = sum x, partial[chunk][1][c] = sum x*y (y = x for variance, or a
// second matrix for the backward dot products). 256 rows per chunk, rows visited in order.
__global__ void colstats_partial_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                        float* __restrict__ partial, int rows, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r0 = blockIdx.y * 256, r1 = min(rows, r0 + 256);
  float s1 = 0.f, s2 = 0.f;
  for (int r = r0; r < r1; ++r) {
    const float x = __bfloat162float(a[static_cast<size_t>(r) * C + c]);
    const float y = __bfloat162float(b[static_cast<size_t>(r) * C + c]);
    s1 += x;
    s2 += x * y;
  }
  partial[(static_cast<size_t>(blockIdx.y) * 2 + 0) * C + c] = s1;
  partial[(static_cast<size_t>(blockIdx.y) * 2 + 1) * C + c] = s2;
}
__global__ void colstats_finish_kernel(const float* __restrict__ partial, int chunks, int C, float* __restrict__ s1,
                                       float* __restrict__ s2) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float a = 0.f, b = 0.f;
  for (int k = 0; k < chunks; ++k) {
    a += partial[(static_cast<size_t>(k) * 2 + 0) * C + c];
    b += partial[(static_cast<size_t>(k) * 2 + 1) * C + c];
  }
  s1[c] = a;
  s2[c] = b;
}

// BatchNorm forward (training): from column sums, mean/var (biased for normalisation), update
// running stats (unbiased variance), y = (x-mean)*inv_std*gamma + beta, optional fused ReLU.
__global__ void bn_prepare_kernel(const float* __restrict__ sum, const float* __restrict__ sumsq, int rows, int C,
                                  float eps, float momentum, float* __restrict__ mean, float* __restrict__ inv_std,
                                  float* __restrict__ run_mean, float* __restrict__ run_var) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float n = static_cast<float>(rows);
  const float m = sum[c] / n;
  const float var = fmaxf(sumsq[c] / n - m * m, 0.f);
  mean[c] = m;
  inv_std[c] = rsqrtf(var + eps);
  if (run_mean) {
    run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * m;
    const float unbiased = rows > 1 ? var * n / (n - 1.f) : var;
    run_var[c] = (1.f - momentum) * run_var[c] + momentum * unbiased;
  }
}
__global__ void bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ mean,
                                const float* __restrict__ inv_std, const float* __restrict__ gamma,
                                const float* __restrict__ beta, __nv_bfloat16* __restrict__ y, size_t total, int C,
                                int relu) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % C);
  float v = (__bfloat162float(x[i]) - mean[c]) * inv_std[c] * gamma[c] + beta[c];
  if (relu) v = fmaxf(v, 0.f);
  y[i] = __float2bfloat16_rn(v);
}
// BatchNorm backward. With xhat = (x-mean)*inv_std, g = dy (already masked by ReLU when fused):
//   dbeta = sum g, dgamma = sum g*xhat, dx = gamma*inv_std/n * (n*g - dbeta - xhat*dgamma)
// sums come from colstats (a = g, b = x): sum g and sum g*x; dgamma = (sum g*x - mean*sum g)*inv_std.
__global__ void bn_bwd_finish_kernel(const float* __restrict__ sum_g, const float* __restrict__ sum_gx,
                                     const float* __restrict__ mean, const float* __restrict__ inv_std, int C,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  dbeta[c] = sum_g[c];
  dgamma[c] = (sum_gx[c] - mean[c] * sum_g[c]) * inv_std[c];
}
__global__ void bn_bwd_dx_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x,
                                 const float* __restrict__ mean, const float* __restrict__ inv_std,
                                 const float* __restrict__ gamma, const float* __restrict__ dgamma,
                                 const float* __restrict__ dbeta, __nv_bfloat16* __restrict__ dx, size_t total,
                                 int C, int rows) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % C);
  const float n = static_cast<float>(rows);
  const float xhat = (__bfloat162float(x[i]) - mean[c]) * inv_std[c];
  const float v = gamma[c] * inv_std[c] / n * (n * __bfloat162float(g[i]) - dbeta[c] - xhat * dgamma[c]);
  dx[i] = __float2bfloat16_rn(v);
}
// g = dy * (y > 0)
__global__ void relu_mask_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                                 __nv_bfloat16* __restrict__ g, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  g[i] = __bfloat162float(y[i]) > 0.f ? dy[i] : __float2bfloat16(0.f);
}
// y = act(x + bias[c])
__global__ void bias_act_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ bias,
                                __nv_bfloat16* __restrict__ y, size_t total, int C, int relu) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = __bfloat162float(x[i]) + (bias ? bias[i % C] : 0.f);
  if (relu) v = fmaxf(v, 0.f);
  y[i] = __float2bfloat16_rn(v);
}

}  // namespace sb

using namespace sb;
#define STREAM static_cast<cudaStream_t>(stream)
#define CHECK_LAUNCH() return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH
static inline unsigned nblk(size_t n) { return static_cast<unsigned>((n + 255) / 256); }

extern "C" int sb_im2col_nhwc(const void* x, void* col, int B, int H, int W, int C, int KH, int KW, int stride,
                              int pad, int OH, int OW, int Kp, void* stream) {
  if (B <= 0 || Kp < KH * KW * C || (Kp & 7)) return SB_ERR_ARG;
  const size_t total = static_cast<size_t>(B) * OH * OW * Kp;
  if ((C & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(col)) & 15) == 0) {
    im2col_nhwc_vec8_kernel<<<nblk(total / 8), 256, 0, STREAM>>>(static_cast<const uint4*>(x), static_cast<uint4*>(col),
                                                                 B, H, W, C / 8, KH, KW, stride, pad, OH, OW, Kp / 8);
    CHECK_LAUNCH();
  }
  im2col_nhwc_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(x),
                                                      static_cast<__nv_bfloat16*>(col), B, H, W, C, KH, KW, stride,
                                                      pad, OH, OW, Kp);
  CHECK_LAUNCH();
}
extern "C" int sb_col2im_nhwc(const void* dcol, void* dx, int B, int H, int W, int C, int KH, int KW, int stride,
                              int pad, int OH, int OW, int Kp, void* stream) {
  if (B <= 0 || Kp < KH * KW * C) return SB_ERR_ARG;
  const size_t total = static_cast<size_t>(B) * H * W * C;
  if ((C & 7) == 0 && (Kp & 7) == 0 && ((reinterpret_cast<uintptr_t>(dcol) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0) {
    col2im_nhwc_vec8_kernel<<<nblk(total / 8), 256, 0, STREAM>>>(static_cast<const uint4*>(dcol),
                                                                 static_cast<uint4*>(dx), B, H, W, C / 8, KH, KW,
                                                                 stride, pad, OH, OW, Kp / 8);
    CHECK_LAUNCH();
  }
  col2im_nhwc_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(dcol),
                                                      static_cast<__nv_bfloat16*>(dx), B, H, W, C, KH, KW, stride,
                                                      pad, OH, OW, Kp);
  CHECK_LAUNCH();
}
extern "C" int sb_maxpool_fwd(const void* x, void* y, void* arg, int B, int H, int W, int C, int k, int stride,
                              int OH, int OW, void* stream) {
  if (B <= 0 || k <= 0 || k > 15) return SB_ERR_ARG;
  const size_t total = static_cast<size_t>(B) * OH * OW * C;
  maxpool_fwd_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(x),
                                                      static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(arg), B,
                                                      H, W, C, k, stride, OH, OW);
  CHECK_LAUNCH();
}
extern "C" int sb_maxpool_bwd(const void* dy, const void* arg, void* dx, int B, int H, int W, int C, int k,
                              int stride, int OH, int OW, void* stream) {
  if (B <= 0 || k <= 0) return SB_ERR_ARG;
  const size_t total = static_cast<size_t>(B) * H * W * C;
  maxpool_bwd_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(dy),
                                                      static_cast<const uint8_t*>(arg),
                                                      static_cast<__nv_bfloat16*>(dx), B, H, W, C, k, stride, OH, OW);
  CHECK_LAUNCH();
}
// partial: 2 * ceil(rows/256) * C floats
extern "C" int sb_colstats(const void* a, const void* b, float* partial, float* s1, float* s2, int rows, int C,
                           void* stream) {
  if (rows <= 0 || C <= 0) return SB_ERR_ARG;
  const int chunks = (rows + 255) / 256;
  dim3 grid((C + 127) / 128, chunks);
  colstats_partial_kernel<<<grid, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(a),
                                                    static_cast<const __nv_bfloat16*>(b), partial, rows, C);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  colstats_finish_kernel<<<(C + 127) / 128, 128, 0, STREAM>>>(partial, chunks, C, s1, s2);
  CHECK_LAUNCH();
}
extern "C" int sb_bn_fwd(const void* x, const float* sum, const float* sumsq, const float* gamma, const float* beta,
                         float* mean, float* inv_std, float* run_mean, float* run_var, void* y, int rows, int C,
                         float eps, float momentum, int relu, int training, void* stream) {
  if (rows <= 0 || C <= 0) return SB_ERR_ARG;
  if (training) {
    bn_prepare_kernel<<<(C + 127) / 128, 128, 0, STREAM>>>(sum, sumsq, rows, C, eps, momentum, mean, inv_std,
                                                           run_mean, run_var);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  const size_t total = static_cast<size_t>(rows) * C;
  bn_apply_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(x), mean, inv_std, gamma, beta,
                                                   static_cast<__nv_bfloat16*>(y), total, C, relu);
  CHECK_LAUNCH();
}
extern "C" int sb_bn_bwd(const void* g, const void* x, const float* sum_g, const float* sum_gx, const float* mean,
                         const float* inv_std, const float* gamma, float* dgamma, float* dbeta, void* dx, int rows,
                         int C, void* stream) {
  if (rows <= 0 || C <= 0) return SB_ERR_ARG;
  bn_bwd_finish_kernel<<<(C + 127) / 128, 128, 0, STREAM>>>(sum_g, sum_gx, mean, inv_std, C, dgamma, dbeta);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  const size_t total = static_cast<size_t>(rows) * C;
  bn_bwd_dx_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(g),
                                                    static_cast<const __nv_bfloat16*>(x), mean, inv_std, gamma,
                                                    dgamma, dbeta, static_cast<__nv_bfloat16*>(dx), total, C, rows);
  CHECK_LAUNCH();
}
extern "C" int sb_relu_mask(const void* dy, const void* y, void* g, size_t total, void* stream) {
  if (total == 0) return SB_ERR_ARG;
  relu_mask_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(dy),
                                                    static_cast<const __nv_bfloat16*>(y),
                                                    static_cast<__nv_bfloat16*>(g), total);
  CHECK_LAUNCH();
}
extern "C" int sb_bias_act(const void* x, const float* bias, void* y, size_t total, int C, int relu, void* stream) {
  if (total == 0 || C <= 0) return SB_ERR_ARG;
  bias_act_kernel<<<nblk(total), 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(x), bias,
                                                   static_cast<__nv_bfloat16*>(y), total, C, relu);
  CHECK_LAUNCH();
}
