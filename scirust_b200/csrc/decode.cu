// Decode-time kernels (small batch, bandwidth-bound): weight-streaming GEMV for bf16 and int8
// per-output-channel weights, paged-KV append, split-KV GQA flash-decode over a paged bf16 cache,
// fused LM-head arg-max with device-side token feedback.
//
// Reference counterparts: one-thread-per-column GEMV and its tiled deterministic variant
// (scirust-cuda/src/bf16_gemv.rs:43-85, bf16_tiled_gemv.rs:43-97), the fused single-query GQA
// kernel (scirust-cuda/src/decode.rs:155-262), the fused LM-head arg-max
// (scirust-cuda/src/bf16_lm_head_argmax.rs:46-176, tie -> lower id), the paged cache semantics of
// scirust-core/src/nn/paged_attention.rs:21-147 and int8 per-channel weights of
// scirust-core/src/quantization.rs:95-190. All reductions have a fixed order (no atomics).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "api.h"

namespace sb {

__device__ __forceinline__ float dbflo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float dbfhi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t dpack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------
// GEMV / skinny GEMM: Y[M,N] (+)= X[M,K] * W[K,N], M <= MB, W streamed once.
// grid = (ceil(N / COLS), splits). A CTA owns COLS output columns and the k range of its split;
// warp w walks rows k0+w, k0+w+8, ...; a lane holds VEC consecutive columns. Partials of the 8
// warps are added in warp order in shared memory, split partials in split order by
// gemv_finish_kernel: the summation tree depends only on (K, splits).
// INT8: W is int8 with one fp32 scale per output column, applied after the sum.
// ---------------------------------------------------------------------------
constexpr int GEMV_KCHUNK = 256;  // rows of X staged in shared memory at a time

// Optional prologue applied to X while it is staged (so the producing kernel disappears):
//   PRO_RMSNORM: x <- bf16(x * rsqrt(mean(x^2) + eps) * norm_w[k]); the row statistic is computed by
//                one warp per row in exactly the order of rmsnorm_fwd_kernel, so fused and unfused
//                paths agree bit for bit.
//   PRO_SWIGLU:  X is a fused [gate | up] row of width 2K: x <- bf16(silu(gate[k]) * up[k]).
enum { PRO_NONE = 0, PRO_RMSNORM = 1, PRO_SWIGLU = 2 };

template <int MB, bool INT8>
__global__ void __launch_bounds__(256)
gemv_kernel(const __nv_bfloat16* __restrict__ X, int ldx, const void* __restrict__ Wv, int ldw, float* __restrict__ part,
            int M, int N, int K, int k_per_split, int prologue, const __nv_bfloat16* __restrict__ norm_w, float eps) {
  constexpr int VEC = INT8 ? 16 : 8;
  constexpr int COLS = 32 * VEC;
  __shared__ float xs[MB][GEMV_KCHUNK];
  __shared__ float buf[256 * VEC];  // cross-warp reduction: [warp][lane][VEC]
  __shared__ float s_inv[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (prologue == PRO_RMSNORM) {
    if (warp < M) {
      const __nv_bfloat16* xr = X + static_cast<size_t>(warp) * ldx;
      float ss = 0.f;
      for (int c = lane * 8; c < K; c += 256) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
        const float f[8] = {dbflo(raw.x), dbfhi(raw.x), dbflo(raw.y), dbfhi(raw.y),
                            dbflo(raw.z), dbfhi(raw.z), dbflo(raw.w), dbfhi(raw.w)};
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_inv[warp] = rsqrtf(ss / static_cast<float>(K) + eps);
    }
    __syncthreads();
  }
  const int col = blockIdx.x * COLS + lane * VEC;
  const int k0 = blockIdx.y * k_per_split;
  const int k1 = min(K, k0 + k_per_split);
  float acc[MB][VEC];
#pragma unroll
  for (int m = 0; m < MB; ++m)
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[m][j] = 0.f;

  for (int kc = k0; kc < k1; kc += GEMV_KCHUNK) {
    const int kn = min(GEMV_KCHUNK, k1 - kc);
    __syncthreads();
    for (int i = threadIdx.x; i < MB * GEMV_KCHUNK; i += 256) {
      const int m = i / GEMV_KCHUNK, kk = i - m * GEMV_KCHUNK;
      float xv = 0.f;
      if (m < M && kk < kn) {
        const int k = kc + kk;
        xv = __bfloat162float(X[static_cast<size_t>(m) * ldx + k]);
        if (prologue == PRO_RMSNORM) {
          xv = __bfloat162float(__float2bfloat16_rn(xv * s_inv[m] * __bfloat162float(norm_w[k])));
        } else if (prologue == PRO_SWIGLU) {
          const float u = __bfloat162float(X[static_cast<size_t>(m) * ldx + K + k]);
          xv = __bfloat162float(__float2bfloat16_rn(xv / (1.f + __expf(-xv)) * u));
        }
      }
      xs[m][kk] = xv;
    }
    __syncthreads();
    if (col < N) {
#pragma unroll 4
      for (int kk = warp; kk < kn; kk += 8) {
        float w[VEC];
        if constexpr (INT8) {
          const int4 raw = *reinterpret_cast<const int4*>(static_cast<const int8_t*>(Wv) +
                                                          static_cast<size_t>(kc + kk) * ldw + col);
          const int32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int b = 0; b < 4; ++b) w[q * 4 + b] = static_cast<float>(static_cast<int8_t>(words[q] >> (8 * b)));
        } else {
          const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(Wv) +
                                                            static_cast<size_t>(kc + kk) * ldw + col);
          w[0] = dbflo(raw.x); w[1] = dbfhi(raw.x); w[2] = dbflo(raw.y); w[3] = dbfhi(raw.y);
          w[4] = dbflo(raw.z); w[5] = dbfhi(raw.z); w[6] = dbflo(raw.w); w[7] = dbfhi(raw.w);
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          const float xv = xs[m][kk];
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[m][j] += xv * w[j];
        }
      }
    }
  }
  // cross-warp reduction in warp order through shared memory, one output row at a time
  __syncthreads();
  for (int m = 0; m < MB; ++m) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) buf[(warp * 32 + lane) * VEC + j] = acc[m][j];
    __syncthreads();
    // thread t sums column t (and t+256 when VEC == 16) over the 8 warps
    for (int c = threadIdx.x; c < COLS; c += 256) {
      const int l = c / VEC, j = c - l * VEC;
      float s = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) s += buf[(w8 * 32 + l) * VEC + j];
      const int gc = blockIdx.x * COLS + c;
      if (m < M && gc < N) part[(static_cast<size_t>(blockIdx.y) * M + m) * N + gc] = s;
    }
    __syncthreads();
  }
}

// out[m,n] = (sum_s part[s,m,n]) * scale[n] (+ residual) -> bf16 and/or fp32
__global__ void gemv_finish_kernel(const float* __restrict__ part, int splits, int M, int N,
                                   const float* __restrict__ scale, const __nv_bfloat16* __restrict__ R, int ldr,
                                   __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ out_f32) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  const int m = i / N, n = i - m * N;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(static_cast<size_t>(k) * M + m) * N + n];
  if (scale) s *= scale[n];
  if (R) s += __bfloat162float(R[static_cast<size_t>(m) * ldr + n]);
  if (out) out[static_cast<size_t>(m) * ldo + n] = __float2bfloat16_rn(s);
  if (out_f32) out_f32[static_cast<size_t>(m) * N + n] = s;
}

// ---------------------------------------------------------------------------
// Paged KV cache. Pool layout: [n_blocks, 2 (k|v), Hkv, page, dh] bf16 per layer.
// block_table[b, i] = physical block of logical block i of sequence b.
// kv_append: copy the (already RoPE'd) k and v heads of `n_tok` tokens from a fused qkv matrix into
// the cache at positions pos[t] of sequence seq_of[t].
// ---------------------------------------------------------------------------
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int H, int Hkv, int dh,
                                 __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_table,
                                 int max_blocks, int page, const int* __restrict__ seq_of,
                                 const int* __restrict__ pos, int n_tok) {
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  const int b = seq_of[t], p = pos[t];
  const int blk = block_table[b * max_blocks + p / page];
  const int slot = p % page;
  const int per = Hkv * dh / 8;  // uint4 per k (or v) row
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * ld + H * dh;
  for (int i = threadIdx.x; i < 2 * per; i += blockDim.x) {
    const int kv = i / per, r = i - kv * per;
    const int h = (r * 8) / dh, d = (r * 8) - h * dh;
    const uint4 v = *reinterpret_cast<const uint4*>(src + kv * Hkv * dh + r * 8);
    __nv_bfloat16* dst = pool + ((((static_cast<size_t>(blk) * 2 + kv) * Hkv + h) * page + slot) * dh + d);
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

// Decode-step fusion of RoPE and the cache append: rotates the q and k heads of each new token in
// place (interleaved pairs, head-local frequency, position pos[t]) and writes the rotated k and the
// v heads into the paged pool. One block per token.
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, int ld, int H, int Hkv, int dh,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_table,
                                      int max_blocks, int page, const int* __restrict__ seq_of,
                                      const int* __restrict__ pos, int n_tok) {
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  const int b = seq_of[t], p = pos[t];
  const int half = dh >> 1;
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld;
  const int n_pairs = (H + Hkv) * half;
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int head = i / half, pr = i - head * half;
    const float c = cos_t[static_cast<size_t>(p) * half + pr], s = sin_t[static_cast<size_t>(p) * half + pr];
    __nv_bfloat16* e = row + head * dh + 2 * pr;
    const float x0 = __bfloat162float(e[0]), x1 = __bfloat162float(e[1]);
    e[0] = __float2bfloat16_rn(x0 * c - x1 * s);
    e[1] = __float2bfloat16_rn(x0 * s + x1 * c);
  }
  __syncthreads();
  const int blk = block_table[b * max_blocks + p / page];
  const int slot = p % page;
  const int per = Hkv * dh / 8;
  const __nv_bfloat16* src = row + H * dh;
  for (int i = threadIdx.x; i < 2 * per; i += blockDim.x) {
    const int kv = i / per, r = i - kv * per;
    const int h = (r * 8) / dh, d = (r * 8) - h * dh;
    const uint4 v = *reinterpret_cast<const uint4*>(src + kv * Hkv * dh + r * 8);
    *reinterpret_cast<uint4*>(pool + ((((static_cast<size_t>(blk) * 2 + kv) * Hkv + h) * page + slot) * dh + d)) = v;
  }
}

// ---------------------------------------------------------------------------
// Split-KV GQA flash-decode. grid = (Hkv, B, n_splits); 128 threads = 4 warps.
// A CTA serves the G = H/Hkv query heads of one kv head for one sequence over the kv positions of
// its split; warp w owns query head w (G <= 4) ... for G > 4 heads are looped. Each warp keeps an
// online softmax (m, l) and a dh-wide accumulator distributed over lanes (dh/32 values per lane).
// K/V rows are read once per CTA into shared memory in tiles of TK positions.
// Partials (m, l, o[dh]) per (b, h, split) are combined in split order by decode_combine_kernel.
// ---------------------------------------------------------------------------
constexpr int DEC_TK = 64;

template <int DH>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ pool,
                   const int* __restrict__ block_table, int max_blocks, int page, const int* __restrict__ seq_len,
                   int H, int Hkv, int n_splits, float scale_log2, float* __restrict__ part_o,
                   float* __restrict__ part_ml) {
  constexpr int VPL = DH / 32;  // accumulator values per lane
  __shared__ __align__(16) __nv_bfloat16 sK[DEC_TK][DH];
  __shared__ __align__(16) __nv_bfloat16 sV[DEC_TK][DH];
  __shared__ float sP[4][DEC_TK];
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = H / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = seq_len[b];
  const int per_split = ((L + n_splits - 1) / n_splits + DEC_TK - 1) / DEC_TK * DEC_TK;
  const int p0 = split * per_split;
  const int p1 = min(L, p0 + per_split);
  for (int g0 = 0; g0 < G; g0 += 4) {
    const int g = g0 + warp;
    const int h = kvh * G + g;
    float qv[VPL];
    if (g < G) {
#pragma unroll
      for (int j = 0; j < VPL; ++j)
        qv[j] = __bfloat162float(q[static_cast<size_t>(b) * ldq + h * DH + lane * VPL + j]) ;
    }
    float m = -1.0e30f, l = 0.f, o[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) o[j] = 0.f;
    for (int t0 = p0; t0 < p1; t0 += DEC_TK) {
      const int tn = min(DEC_TK, p1 - t0);
      __syncthreads();
      for (int i = threadIdx.x; i < tn * (DH / 8); i += 128) {
        const int r = i / (DH / 8), c = (i - r * (DH / 8)) * 8;
        const int pos = t0 + r;
        const int blk = block_table[b * max_blocks + pos / page];
        const size_t base = (((static_cast<size_t>(blk) * 2) * Hkv + kvh) * page + pos % page) * DH + c;
        const size_t vofs = static_cast<size_t>(Hkv) * page * DH;
        *reinterpret_cast<uint4*>(&sK[r][c]) = *reinterpret_cast<const uint4*>(pool + base);
        *reinterpret_cast<uint4*>(&sV[r][c]) = *reinterpret_cast<const uint4*>(pool + base + vofs);
      }
      __syncthreads();
      if (g < G) {
        // scores: each lane takes positions lane, lane+32 ...; dot over dh needs all of q: use shuffles
        float mx = -1.0e30f;
        for (int r = 0; r < tn; ++r) {
          float partial = 0.f;
#pragma unroll
          for (int j = 0; j < VPL; ++j) partial += qv[j] * __bfloat162float(sK[r][lane * VPL + j]);
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, off);
          if (lane == 0) sP[warp][r] = partial * scale_log2;
          mx = fmaxf(mx, partial * scale_log2);
        }
        __syncwarp();
        const float m_new = fmaxf(m, mx);
        const float alpha = exp2f(m - m_new);
        float rowsum = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) o[j] *= alpha;
        for (int r = 0; r < tn; ++r) {
          const float pr = exp2f(sP[warp][r] - m_new);
          rowsum += pr;
#pragma unroll
          for (int j = 0; j < VPL; ++j) o[j] += pr * __bfloat162float(sV[r][lane * VPL + j]);
        }
        l = l * alpha + rowsum;
        m = m_new;
        __syncwarp();
      }
    }
    if (g < G) {
      const size_t idx = (static_cast<size_t>(b) * H + h) * n_splits + split;
#pragma unroll
      for (int j = 0; j < VPL; ++j) part_o[idx * DH + lane * VPL + j] = o[j];
      if (lane == 0) {
        part_ml[idx * 2] = m;
        part_ml[idx * 2 + 1] = l;
      }
    }
  }
}

// Combine split partials in split order 0..S-1 and write bf16 output [B, H*dh].
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      int n_splits, int dh, __nv_bfloat16* __restrict__ out, int ldo, int H) {
  const int bh = blockIdx.x;  // b*H + h
  const int b = bh / H, h = bh - b * H;
  const int d = threadIdx.x;
  if (d >= dh) return;
  float m = -1.0e30f;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(static_cast<size_t>(bh) * n_splits + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const size_t idx = static_cast<size_t>(bh) * n_splits + s;
    const float w = exp2f(part_ml[idx * 2] - m);
    l += part_ml[idx * 2 + 1] * w;
    o += part_o[idx * dh + d] * w;
  }
  out[static_cast<size_t>(b) * ldo + h * dh + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
}

// ---------------------------------------------------------------------------
// Arg-max over logits rows with the reference's tie rule (first maximum wins; a NaN never wins
// against a number because `v > best` is false for NaN, decode.rs:107-114), two stages.
// Stage 1: each CTA scans a slab of `cols_per_cta` columns of one row -> (value, index).
// Stage 2: one CTA per row picks the best slab result, lower index on ties, and writes the token
// to `out_tokens[row]` (int64, the device-side feedback buffer) and optionally appends it to
// `generated[row, step]`.
// ---------------------------------------------------------------------------
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int V, int cols_per_cta,
                                      float* __restrict__ pval, int* __restrict__ pidx) {
  __shared__ float sv[256];
  __shared__ int si[256];
  const int row = blockIdx.y, slab = blockIdx.x;
  const int c0 = slab * cols_per_cta, c1 = min(V, c0 + cols_per_cta);
  const float* lr = logits + static_cast<size_t>(row) * V;
  float best = -INFINITY;
  int bi = c0;
  bool have = false;
  for (int c = c0 + threadIdx.x; c < c1; c += 256) {
    const float v = lr[c];
    if (!have) { best = v; bi = c; have = true; }
    else if (v > best) { best = v; bi = c; }
  }
  sv[threadIdx.x] = have ? best : -INFINITY;
  si[threadIdx.x] = have ? bi : 0x7fffffff;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float a = sv[threadIdx.x], bb = sv[threadIdx.x + s];
      const int ia = si[threadIdx.x], ib = si[threadIdx.x + s];
      // keep the larger value; on equal values (or NaN on either side) keep the lower index
      const bool take_b = (bb > a) || (!(a > bb) && !(bb > a) && ib < ia);
      if (take_b) { sv[threadIdx.x] = bb; si[threadIdx.x] = ib; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    pval[row * gridDim.x + slab] = sv[0];
    pidx[row * gridDim.x + slab] = si[0];
  }
}
__global__ void argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int n_slabs,
                                    int64_t* __restrict__ out_tokens, int64_t* __restrict__ generated,
                                    int gen_stride, int step) {
  const int row = blockIdx.x;
  if (threadIdx.x != 0) return;
  float best = pval[row * n_slabs];
  int bi = pidx[row * n_slabs];
  for (int s = 1; s < n_slabs; ++s) {
    const float v = pval[row * n_slabs + s];
    const int i = pidx[row * n_slabs + s];
    if (v > best || (!(best > v) && !(v > best) && i < bi)) { best = v; bi = i; }
  }
  if (bi == 0x7fffffff) bi = 0;
  out_tokens[row] = bi;
  if (generated) generated[static_cast<size_t>(row) * gen_stride + step] = bi;
}

// Per-output-channel symmetric int8 quantisation of W [K, N] (x.W layout): scale[n] = max|W[:,n]|/127
// (1 when the column is zero), q = clamp(round(W/scale), -128, 127)   (quantization.rs:95-125).
__global__ void quant_colmax_kernel(const __nv_bfloat16* __restrict__ W, int K, int N, int ldw,
                                    float* __restrict__ scale) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float mx = 0.f;
  for (int k = 0; k < K; ++k) mx = fmaxf(mx, fabsf(__bfloat162float(W[static_cast<size_t>(k) * ldw + n])));
  scale[n] = mx == 0.f ? 1.f : mx / 127.f;
}
__global__ void quant_apply_kernel(const __nv_bfloat16* __restrict__ W, int K, int N, int ldw,
                                   const float* __restrict__ scale, int8_t* __restrict__ Q) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<size_t>(K) * N) return;
  const size_t k = i / N;
  const int n = static_cast<int>(i - k * N);
  const float v = roundf(__bfloat162float(W[k * ldw + n]) / scale[n]);  // roundf: half away from zero
  Q[i] = static_cast<int8_t>(fminf(fmaxf(v, -128.f), 127.f));
}
// bf16 copy of an int8 matrix times its column scales (used to feed the tensor-core GEMM in prefill)
__global__ void dequant_kernel(const int8_t* __restrict__ Q, const float* __restrict__ scale, int K, int N,
                               __nv_bfloat16* __restrict__ W) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<size_t>(K) * N) return;
  const int n = static_cast<int>(i % N);
  W[i] = __float2bfloat16_rn(static_cast<float>(Q[i]) * scale[n]);
}

}  // namespace sb

using namespace sb;
#define STREAM static_cast<cudaStream_t>(stream)
#define CHECK_LAUNCH() return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH

template <bool INT8>
static int launch_gemv(const void* X, int ldx, const void* W, int ldw, float* part, int M, int N, int K, int splits,
                       int kps, int pro, const void* nw, float eps, cudaStream_t s) {
  constexpr int COLS = INT8 ? 512 : 256;
  dim3 grid((N + COLS - 1) / COLS, splits);
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
  if (M <= 1) gemv_kernel<1, INT8><<<grid, 256, 0, s>>>(x, ldx, W, ldw, part, M, N, K, kps, pro, static_cast<const __nv_bfloat16*>(nw), eps);
  else if (M <= 2) gemv_kernel<2, INT8><<<grid, 256, 0, s>>>(x, ldx, W, ldw, part, M, N, K, kps, pro, static_cast<const __nv_bfloat16*>(nw), eps);
  else if (M <= 4) gemv_kernel<4, INT8><<<grid, 256, 0, s>>>(x, ldx, W, ldw, part, M, N, K, kps, pro, static_cast<const __nv_bfloat16*>(nw), eps);
  else if (M <= 8) gemv_kernel<8, INT8><<<grid, 256, 0, s>>>(x, ldx, W, ldw, part, M, N, K, kps, pro, static_cast<const __nv_bfloat16*>(nw), eps);
  else return SB_ERR_ARG;
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// Y[M,N] = X[M,K] * W[K,N] (* scale[n]) (+ R). M <= 8 per call (callers loop over row groups).
// W bf16 (is_int8 == 0) or int8 with fp32 column scales. workspace: splits*M*N floats.
// Returns the number of k-splits used through *splits_out when splits == 0 (auto).
// prologue: 0 none, 1 RMSNorm of X with gain norm_w (K must be a multiple of 8), 2 SwiGLU over a
// fused [gate | up] X of row width 2K.
extern "C" int sb_gemv(const void* X, int ldx, const void* W, int ldw, const float* scale, const void* R, int ldr,
                       void* out_bf16, int ldo, float* out_f32, int M, int N, int K, int is_int8, int splits,
                       float* workspace, int prologue, const void* norm_w, float eps, void* stream) {
  if (M <= 0 || M > 8 || N <= 0 || K <= 0 || (N & 7) || (is_int8 && (N & 15))) return SB_ERR_ARG;
  if (prologue < 0 || prologue > 2 || (prologue == 1 && (!norm_w || (K & 7) || (ldx & 7)))) return SB_ERR_ARG;
  if (splits < 1) splits = 1;
  int kps = ((K + splits - 1) / splits + 7) / 8 * 8;
  splits = (K + kps - 1) / kps;
  int rc = is_int8 ? launch_gemv<true>(X, ldx, W, ldw, workspace, M, N, K, splits, kps, prologue, norm_w, eps, STREAM)
                   : launch_gemv<false>(X, ldx, W, ldw, workspace, M, N, K, splits, kps, prologue, norm_w, eps, STREAM);
  if (rc) return rc;
  gemv_finish_kernel<<<(M * N + 255) / 256, 256, 0, STREAM>>>(workspace, splits, M, N, scale,
                                                             static_cast<const __nv_bfloat16*>(R), ldr,
                                                             static_cast<__nv_bfloat16*>(out_bf16), ldo, out_f32);
  CHECK_LAUNCH();
}

extern "C" int sb_kv_append(const void* qkv, int ld, int H, int Hkv, int dh, void* pool, const int* block_table,
                            int max_blocks, int page, const int* seq_of, const int* pos, int n_tok, void* stream) {
  if (n_tok <= 0 || (dh & 7)) return SB_ERR_ARG;
  kv_append_kernel<<<n_tok, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(qkv), ld, H, Hkv, dh,
                                              static_cast<__nv_bfloat16*>(pool), block_table, max_blocks, page,
                                              seq_of, pos, n_tok);
  CHECK_LAUNCH();
}

extern "C" int sb_rope_kv_append(void* qkv, int ld, int H, int Hkv, int dh, const float* cos_t, const float* sin_t,
                                 void* pool, const int* block_table, int max_blocks, int page, const int* seq_of,
                                 const int* pos, int n_tok, void* stream) {
  if (n_tok <= 0 || (dh & 7)) return SB_ERR_ARG;
  rope_kv_append_kernel<<<n_tok, 256, 0, STREAM>>>(static_cast<__nv_bfloat16*>(qkv), ld, H, Hkv, dh, cos_t, sin_t,
                                                   static_cast<__nv_bfloat16*>(pool), block_table, max_blocks, page,
                                                   seq_of, pos, n_tok);
  CHECK_LAUNCH();
}

// q: bf16 [B, ldq] (H*dh used, RoPE'd); out: bf16 [B, ldo]. part_o: B*H*n_splits*dh floats,
// part_ml: B*H*n_splits*2 floats (scratch).
extern "C" int sb_decode_attention(const void* q, int ldq, const void* pool, const int* block_table, int max_blocks,
                                   int page, const int* seq_len, int B, int H, int Hkv, int dh, int n_splits,
                                   float scale, float* part_o, float* part_ml, void* out, int ldo, void* stream) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) || (dh != 64 && dh != 128) || n_splits < 1) return SB_ERR_ARG;
  dim3 grid(Hkv, B, n_splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (dh == 64)
    decode_attn_kernel<64><<<grid, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(q), ldq,
                                                     static_cast<const __nv_bfloat16*>(pool), block_table,
                                                     max_blocks, page, seq_len, H, Hkv, n_splits, sl2, part_o,
                                                     part_ml);
  else
    decode_attn_kernel<128><<<grid, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(q), ldq,
                                                      static_cast<const __nv_bfloat16*>(pool), block_table,
                                                      max_blocks, page, seq_len, H, Hkv, n_splits, sl2, part_o,
                                                      part_ml);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  decode_combine_kernel<<<B * H, dh, 0, STREAM>>>(part_o, part_ml, n_splits, dh, static_cast<__nv_bfloat16*>(out),
                                                  ldo, H);
  CHECK_LAUNCH();
}

// logits: fp32 [rows, V]. pval/pidx: rows * ceil(V/4096) scratch. out_tokens: int64 [rows].
extern "C" int sb_argmax(const float* logits, int rows, int V, float* pval, int* pidx, int64_t* out_tokens,
                         int64_t* generated, int gen_stride, int step, void* stream) {
  if (rows <= 0 || V <= 0) return SB_ERR_ARG;
  const int cpc = 4096;
  const int slabs = (V + cpc - 1) / cpc;
  argmax_partial_kernel<<<dim3(slabs, rows), 256, 0, STREAM>>>(logits, V, cpc, pval, pidx);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  argmax_final_kernel<<<rows, 32, 0, STREAM>>>(pval, pidx, slabs, out_tokens, generated, gen_stride, step);
  CHECK_LAUNCH();
}

extern "C" int sb_quantize_per_channel(const void* W, int K, int N, int ldw, float* scale, void* Q, void* stream) {
  if (K <= 0 || N <= 0) return SB_ERR_ARG;
  quant_colmax_kernel<<<(N + 127) / 128, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(W), K, N, ldw, scale);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  const size_t n = static_cast<size_t>(K) * N;
  quant_apply_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM>>>(
      static_cast<const __nv_bfloat16*>(W), K, N, ldw, scale, static_cast<int8_t*>(Q));
  CHECK_LAUNCH();
}
extern "C" int sb_dequantize(const void* Q, const float* scale, int K, int N, void* W, void* stream) {
  const size_t n = static_cast<size_t>(K) * N;
  if (n == 0) return SB_ERR_ARG;
  dequant_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM>>>(static_cast<const int8_t*>(Q), scale,
                                                                            K, N, static_cast<__nv_bfloat16*>(W));
  CHECK_LAUNCH();
}
