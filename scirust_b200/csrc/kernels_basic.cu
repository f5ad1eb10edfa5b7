// Bandwidth-bound training kernels: RMSNorm fwd/bwd, RoPE fwd/bwd, SwiGLU fwd/bwd,
// embedding gather / deterministic scatter-add, fused softmax-cross-entropy
// (loss + gradient in place), deterministic sum of squares, fused AdamW over a flat
// parameter buffer, casts. bf16 storage, fp32 math, RNE rounding on store.
//
// Semantics follow the reference's scalar CUDA-C kernels
// (scirust-cuda/src/chain.rs: rmsnorm_fast :423, rope :225/:350, swiglu :55/:278,
// embed :247/:579, ce_loss_grad :637, adamw_norm :707, sumsq :742/:759) but the
// shapes are different: 16-byte vector accesses, warp-per-row reductions with a
// fixed shuffle tree (bitwise repeatable, no atomics), one launch per flat buffer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "api.h"

namespace sb {

__device__ __forceinline__ float bflo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bfhi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t packbf(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bflo(v.x); f[1] = bfhi(v.x); f[2] = bflo(v.y); f[3] = bfhi(v.y);
  f[4] = bflo(v.z); f[5] = bfhi(v.z); f[6] = bflo(v.w); f[7] = bfhi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(packbf(f[0], f[1]), packbf(f[2], f[3]), packbf(f[4], f[5]), packbf(f[6], f[7]));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * w. One warp per row.
// Optionally stores inv_rms (fp32 per row) for the backward pass.
// ---------------------------------------------------------------------------
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ inv_rms, int rows, int cols,
                                   int ldx, int ldy, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  // eight interleaved accumulators (iteration i of the lane goes to accumulator i % 8), added in
  // index order: more loads in flight, and the same association as the fused prologue of the decode
  // GEMV, which spreads the eight accumulators over eight warps
  float acc[8];
#pragma unroll
  for (int a = 0; a < 8; ++a) acc[a] = 0.f;
  for (int c0 = lane * 8; c0 < cols; c0 += 8 * 256) {
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int c = c0 + a * 256;
      if (c < cols) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + c), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[a] += f[j] * f[j];
      }
    }
  }
  float ss = acc[0];
#pragma unroll
  for (int a = 1; a < 8; ++a) ss += acc[a];
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / static_cast<float>(cols) + eps);
  if (inv_rms && lane == 0) inv_rms[row] = inv;
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * ldy;
  for (int c = lane * 8; c < cols; c += 256) {
    float f[8], g[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c), f);
    unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * inv * g[j];
    *reinterpret_cast<uint4*>(yr + c) = pack8(f);
  }
}

// RMSNorm backward, input gradient. With g = dy*w and r = inv_rms:
//   dx = r * (g - x * r^2 * mean(g*x))   (+ optional residual-stream gradient `dres`)
__global__ void rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ inv_rms,
                                      const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                      int rows, int cols) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const size_t off = static_cast<size_t>(row) * cols;
  float dot = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float a[8], b[8], g[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + off + c), a);
    unpack8(*reinterpret_cast<const uint4*>(x + off + c), b);
    unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += a[j] * g[j] * b[j];
  }
  dot = warp_sum(dot);
  const float r = inv_rms[row];
  const float k = r * r * dot / static_cast<float>(cols);
  for (int c = lane * 8; c < cols; c += 256) {
    float a[8], b[8], g[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + off + c), a);
    unpack8(*reinterpret_cast<const uint4*>(x + off + c), b);
    unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = r * (a[j] * g[j] - b[j] * k);
    if (dres) {
      float d[8];
      unpack8(*reinterpret_cast<const uint4*>(dres + off + c), d);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += d[j];
    }
    *reinterpret_cast<uint4*>(dx + off + c) = pack8(o);
  }
}

// The same for rows of NV * 256 columns (NV <= 8): dy and x of the row stay in registers, all loads are issued
// before the first use, and the sums run in the order of the general kernel (same bits).
template <int NV>
__global__ void rmsnorm_bwd_dx_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                          const __nv_bfloat16* __restrict__ w, const float* __restrict__ inv_rms,
                                          const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                          int rows) {
  constexpr int cols = NV * 256;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const size_t off = static_cast<size_t>(row) * cols;
  uint4 va[NV], vb[NV], vg[NV], vd[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane * 8 + i * 256;
    va[i] = *reinterpret_cast<const uint4*>(dy + off + c);
    vb[i] = *reinterpret_cast<const uint4*>(x + off + c);
    vg[i] = *reinterpret_cast<const uint4*>(w + c);
    if (dres) vd[i] = *reinterpret_cast<const uint4*>(dres + off + c);
  }
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float a[8], b[8], g[8];
    unpack8(va[i], a); unpack8(vb[i], b); unpack8(vg[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += a[j] * g[j] * b[j];
  }
  dot = warp_sum(dot);
  const float r = inv_rms[row];
  const float k = r * r * dot / static_cast<float>(cols);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float a[8], b[8], g[8], o[8];
    unpack8(va[i], a); unpack8(vb[i], b); unpack8(vg[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = r * (a[j] * g[j] - b[j] * k);
    if (dres) {
      float d[8];
      unpack8(vd[i], d);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += d[j];
    }
    *reinterpret_cast<uint4*>(dx + off + lane * 8 + i * 256) = pack8(o);
  }
}

// RMSNorm gain gradient, stage 1: partial[ry][j] = sum over the rows of chunk ry of
// dy*x*inv_rms, rows visited in ascending order by each warp, warps combined in warp
// order. Stage 2 (colsum_finish_kernel) adds the chunks in chunk order.
__global__ void rmsnorm_bwd_dw_partial_kernel(const __nv_bfloat16* __restrict__ dy,
                                              const __nv_bfloat16* __restrict__ x,
                                              const float* __restrict__ inv_rms, float* __restrict__ partial,
                                              int rows, int cols, int rows_per_chunk) {
  __shared__ float red[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < cols) {
    // four rows of this warp in flight; the adds keep the row order
    for (int r = r0 + warp; r < r1; r += 32) {
      uint4 va[4], vb[4];
      float iv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 8 * u;
        if (rr < r1) {
          va[u] = *reinterpret_cast<const uint4*>(dy + static_cast<size_t>(rr) * cols + c);
          vb[u] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(rr) * cols + c);
          iv[u] = inv_rms[rr];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r + 8 * u < r1) {
          float a[8], b[8];
          unpack8(va[u], a);
          unpack8(vb[u], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += a[j] * b[j] * iv[u];
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int t = threadIdx.x;
  float s = 0.f;
#pragma unroll
  for (int wdx = 0; wdx < 8; ++wdx) s += red[wdx][t];
  const int col = blockIdx.x * 256 + t;
  if (col < cols) partial[static_cast<size_t>(blockIdx.y) * cols + col] = s;
}


// Generic fixed-order column sum finish: out[j] = sum_k partial[k][j] (k ascending);
// writes fp32 and/or bf16.
__global__ void colsum_finish_kernel(const float* __restrict__ partial, int chunks, int cols,
                                     float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= cols) return;
  float s = 0.f;
  for (int k = 0; k < chunks; ++k) s += partial[static_cast<size_t>(k) * cols + j];
  if (out_f32) out_f32[j] = s;
  if (out_bf16) out_bf16[j] = __float2bfloat16_rn(s);
}

// ---------------------------------------------------------------------------
// RoPE on interleaved pairs, head-local frequency, rotate in place. `x` points at a
// [rows, ld] matrix whose first n_heads*dh columns are rotated (q heads then k heads
// of a fused qkv buffer). Table: cos/sin fp32 [max_pos, dh/2]. sign=+1 forward,
// -1 backward (the transpose of a rotation is the rotation by the negative angle).
// pos = positions[r] if given, else (r % seq_len) + offset.
// ---------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, int ld, int rows, int n_heads, int dh, int seq_len,
                            int offset, const int* __restrict__ positions, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, float sign) {
  const int half = dh >> 1;
  const int quads_per_row = n_heads * (half >> 2);  // 4 pairs (8 bf16 = 16 B) per thread
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * quads_per_row) return;
  const int r = static_cast<int>(idx / quads_per_row);
  const int qd = static_cast<int>(idx - static_cast<size_t>(r) * quads_per_row);
  const int head = qd / (half >> 2);
  const int p0 = (qd - head * (half >> 2)) * 4;  // first pair index inside the head
  const int pos = positions ? positions[r] : (r % seq_len) + offset;
  __nv_bfloat16* ptr = x + static_cast<size_t>(r) * ld + head * dh + p0 * 2;
  float f[8];
  unpack8(*reinterpret_cast<const uint4*>(ptr), f);
  const float4 c = *reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(pos) * half + p0);
  float4 s = *reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(pos) * half + p0);
  s.x *= sign; s.y *= sign; s.z *= sign; s.w *= sign;
  float o[8];
  o[0] = f[0] * c.x - f[1] * s.x; o[1] = f[0] * s.x + f[1] * c.x;
  o[2] = f[2] * c.y - f[3] * s.y; o[3] = f[2] * s.y + f[3] * c.y;
  o[4] = f[4] * c.z - f[5] * s.z; o[5] = f[4] * s.z + f[5] * c.z;
  o[6] = f[6] * c.w - f[7] * s.w; o[7] = f[6] * s.w + f[7] * c.w;
  *reinterpret_cast<uint4*>(ptr) = pack8(o);
}

// ---------------------------------------------------------------------------
// SwiGLU over a fused [gate | up] activation: gu is [rows, 2*ff], h is [rows, ff].
// ---------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, int rows,
                                  int ff) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = ff >> 3;
  if (idx >= static_cast<size_t>(rows) * per_row) return;
  const size_t r = idx / per_row;
  const int c = static_cast<int>(idx - r * per_row) * 8;
  float g[8], u[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * ff + c), g);
  unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * ff + ff + c), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  *reinterpret_cast<uint4*>(h + r * ff + c) = pack8(o);
}

// dgu = [dh*u*silu'(g) | dh*silu(g)], silu'(g) = s*(1 + g*(1-s)), s = sigmoid(g).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, int rows, int ff) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = ff >> 3;
  if (idx >= static_cast<size_t>(rows) * per_row) return;
  const size_t r = idx / per_row;
  const int c = static_cast<int>(idx - r * per_row) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * ff + c), g);
  unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * ff + ff + c), u);
  unpack8(*reinterpret_cast<const uint4*>(dh + r * ff + c), d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float s = 1.f / (1.f + __expf(-g[j]));
    dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
    du[j] = d[j] * g[j] * s;
  }
  *reinterpret_cast<uint4*>(dgu + r * 2 * ff + c) = pack8(dg);
  *reinterpret_cast<uint4*>(dgu + r * 2 * ff + ff + c) = pack8(du);
}

// out = a + b (bf16), 8 elements per thread.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, size_t n8) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float x[8], y[8];
  unpack8(reinterpret_cast<const uint4*>(a)[i], x);
  unpack8(reinterpret_cast<const uint4*>(b)[i], y);
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] += y[j];
  reinterpret_cast<uint4*>(out)[i] = pack8(x);
}

// ---------------------------------------------------------------------------
// Embedding gather (out row i = table row tokens[i]; ids clamped to the table) and
// its deterministic backward: tokens are sorted (stable) on the device beforehand;
// one block per sorted position, only segment heads do work and add their segment's
// rows in sorted order into the table gradient (which may already hold the tied
// LM-head weight gradient).
// ---------------------------------------------------------------------------
__global__ void embed_fwd_kernel(const __nv_bfloat16* __restrict__ table, const int64_t* __restrict__ tokens,
                                 __nv_bfloat16* __restrict__ out, int n, int d, int vocab) {
  const int i = blockIdx.x;
  if (i >= n) return;
  int64_t t = tokens[i];
  if (t < 0) t = 0;
  if (t >= vocab) t = vocab - 1;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(t) * d);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(i) * d);
  for (int c = threadIdx.x; c < (d >> 3); c += blockDim.x) dst[c] = src[c];
}

__global__ void embed_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const int64_t* __restrict__ sorted_tok,
                                 const int64_t* __restrict__ perm, __nv_bfloat16* __restrict__ dtable, int n, int d,
                                 int vocab, int accumulate) {
  const int i = blockIdx.x;
  if (i >= n) return;
  const int64_t tok = sorted_tok[i];
  if (i > 0 && sorted_tok[i - 1] == tok) return;  // not a segment head
  int64_t t = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  for (int c = threadIdx.x; c < (d >> 3); c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4* dst = reinterpret_cast<uint4*>(dtable + static_cast<size_t>(t) * d) + c;
    if (accumulate) unpack8(*dst, acc);
    for (int j = i; j < n && sorted_tok[j] == tok; ++j) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(dy + static_cast<size_t>(perm[j]) * d)[c], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
    *dst = pack8(acc);
  }
}

// ---------------------------------------------------------------------------
// Fused softmax cross-entropy. One block per row: pass 1 online (max, sum) with a
// fixed combine tree, pass 2 writes d = (softmax - onehot) * grad_scale over the
// logits in place (or to `dlogits`). Target ids >= cols clamp to cols-1; rows whose
// target is negative contribute zero loss and zero gradient (ignore index).
// ---------------------------------------------------------------------------
struct MaxSum { float m, s; };
__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  const float m = fmaxf(a.m, b.m);
  MaxSum r;
  r.m = m;
  r.s = a.s * __expf(a.m - m) + b.s * __expf(b.m - m);
  return r;
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
ce_fwd_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                  float* __restrict__ loss_rows, __nv_bfloat16* __restrict__ dlogits, int rows, int cols, int ld,
                  float grad_scale) {
  __shared__ MaxSum red[THREADS / 32];
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(r) * ld;
  MaxSum acc;
  acc.m = -3.0e38f;
  acc.s = 0.f;
  for (int c = tid * 8; c < cols; c += THREADS * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(lr + c), f);
    float mx = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, f[j]);
    const float m = fmaxf(acc.m, mx);
    float s = acc.s * __expf(acc.m - m);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    acc.m = m;
    acc.s = s;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other;
    other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
    // combine in a lane-symmetric way so every lane holds identical bits
    acc = (lane & o) ? ms_combine(other, acc) : ms_combine(acc, other);
  }
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  MaxSum tot = red[0];
#pragma unroll
  for (int w = 1; w < THREADS / 32; ++w) tot = ms_combine(tot, red[w]);
  int64_t tgt = targets[r];
  const bool ignore = tgt < 0;
  if (tgt >= cols) tgt = cols - 1;
  if (tid == 0) {
    loss_rows[r] = ignore ? 0.f : -(__bfloat162float(lr[tgt]) - tot.m) + logf(tot.s);
  }
  if (!dlogits) return;
  __nv_bfloat16* dr = dlogits + static_cast<size_t>(r) * ld;
  const float inv = 1.f / tot.s;
  const float gs = ignore ? 0.f : grad_scale;
  for (int c = tid * 8; c < cols; c += THREADS * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(lr + c), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - tot.m) * inv;
      if (c + j == tgt) p -= 1.f;
      f[j] = p * gs;
    }
    *reinterpret_cast<uint4*>(dr + c) = pack8(f);
  }
}

// ---------------------------------------------------------------------------
// Vocabulary-parallel softmax cross-entropy: every rank holds the logits of its vocabulary shard
// [v0, v0 + cols). Phase 1 writes per-row (max, sum exp(x - max), target logit or 0) of the shard;
// the ranks combine the three numbers; phase 2 turns the shard's logits into
// (exp(x - lse) - onehot) * grad_scale with the global log-sum-exp. Rows with a negative target
// contribute nothing.
// ---------------------------------------------------------------------------
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
ce_shard_stats_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                      float* __restrict__ stats, int rows, int cols, int ld, int v0) {
  __shared__ MaxSum red[THREADS / 32];
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(r) * ld;
  MaxSum acc;
  acc.m = -3.0e38f;
  acc.s = 0.f;
  for (int c = tid * 8; c < cols; c += THREADS * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(lr + c), f);
    float mx = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, f[j]);
    const float m = fmaxf(acc.m, mx);
    float s = acc.s * __expf(acc.m - m);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    acc.m = m;
    acc.s = s;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other;
    other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
    acc = (lane & o) ? ms_combine(other, acc) : ms_combine(acc, other);
  }
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (tid == 0) {
    MaxSum tot = red[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; ++w) tot = ms_combine(tot, red[w]);
    const int64_t tgt = targets[r] - v0;
    stats[r * 3 + 0] = tot.m;
    stats[r * 3 + 1] = tot.s;
    stats[r * 3 + 2] = (tgt >= 0 && tgt < cols && targets[r] >= 0) ? __bfloat162float(lr[tgt]) : 0.f;
  }
}

__global__ void __launch_bounds__(512)
ce_shard_grad_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                     const float* __restrict__ lse, __nv_bfloat16* __restrict__ dlogits, int rows, int cols, int ld,
                     int v0, float grad_scale) {
  const int r = blockIdx.x;
  if (r >= rows) return;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(r) * ld;
  __nv_bfloat16* dr = dlogits + static_cast<size_t>(r) * ld;
  const bool ignore = targets[r] < 0;
  const int64_t tgt = targets[r] - v0;
  const float l = lse[r];
  const float gs = ignore ? 0.f : grad_scale;
  for (int c = threadIdx.x * 8; c < cols; c += 512 * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(lr + c), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - l);
      if (c + j == tgt) p -= 1.f;
      f[j] = p * gs;
    }
    *reinterpret_cast<uint4*>(dr + c) = pack8(f);
  }
}

// ---------------------------------------------------------------------------
// Deterministic sum of squares of a flat bf16 or fp32 buffer: one fp32 partial per
// block (fixed tree), then a single block adds the partials in a fixed strided order.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p, size_t i) { return p[i]; }

// Elements summed by one block of sumsq_partial_kernel (= one partial): 256 threads x 16 strided reads.
// sb_sumsq and sb_sumsq_no_alloc both size their launch from this one constant.
constexpr size_t kSumsqElemsPerPartial = 4096;

template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ g, size_t n, float* __restrict__ partials) {
  __shared__ float red[8];
  float v = 0.f;
  const size_t base = static_cast<size_t>(blockIdx.x) * kSumsqElemsPerPartial;
#pragma unroll 4
  for (int k = 0; k < static_cast<int>(kSumsqElemsPerPartial / 256); ++k) {
    const size_t i = base + k * 256 + threadIdx.x;
    if (i < n) {
      const float x = ld_as_float<T>(g, i);
      v += x * x;
    }
  }
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w];
    partials[blockIdx.x] = s;
  }
}
__global__ void sumsq_finish_kernel(const float* __restrict__ partials, int n_partials, float* __restrict__ out,
                                    int accumulate) {
  __shared__ float red[8];
  float v = 0.f;
  for (int i = threadIdx.x; i < n_partials; i += 256) v += partials[i];
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w];
    out[0] = accumulate ? out[0] + s : s;
  }
}

// ---------------------------------------------------------------------------
// Fused AdamW / Adam / SGD-momentum over a flat parameter buffer.
// fp32 master p, fp32 m/v, gradient bf16 or fp32, fresh bf16 copy of p written for the
// next forward. The clip factor is derived on the device from grad_sumsq[0]
// (sum of squares of the whole model's gradient): non-finite => the update is
// skipped, norm > max_grad_norm => gradients are scaled by max/norm. Elements at
// index >= decay_end (norm gains, biases) take no weight decay.
// mode: 0 = AdamW (decoupled decay), 1 = Adam (L2 decay folded into g), 2 = SGD
// with momentum (m is the velocity, v unused).
// ---------------------------------------------------------------------------
// One element of the update; shared by the scalar and the 4-wide kernels so both give the same bits.
__device__ __forceinline__ void optim_update_one(float& pi, float& mi, float& vi, float g, float wdi, float lr,
                                                 float b1, float b2, float eps, float bc1, float bc2, int mode) {
  if (mode == 2) {
    if (wdi > 0.f) g += wdi * pi;
    const float vel = b1 * mi + g;
    mi = vel;
    pi -= lr * vel;
  } else {
    if (mode == 1 && wdi > 0.f) g += wdi * pi;
    mi = b1 * mi + (1.f - b1) * g;
    vi = b2 * vi + (1.f - b2) * g * g;
    const float mhat = mi / bc1;
    const float vhat = vi / bc2;
    if (mode == 0) pi -= lr * (mhat / (sqrtf(vhat) + eps) + wdi * pi);
    else pi -= lr * mhat / (sqrtf(vhat) + eps);
  }
}

__device__ __forceinline__ bool optim_clip_scale(const float* grad_sumsq, float max_grad_norm, float grad_scale,
                                                 float& scale) {
  scale = grad_scale;
  if (grad_sumsq) {
    const float sq = grad_sumsq[0] * grad_scale * grad_scale;
    const float norm = sqrtf(sq);
    if (!(sq >= 0.f) || sq > 3.0e38f) return false;  // NaN / inf gradient: skip the whole update
    if (max_grad_norm > 0.f && norm > max_grad_norm) scale *= max_grad_norm / norm;
  }
  return true;
}

template <typename G>
__global__ void optim_step_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                  const G* __restrict__ grad, __nv_bfloat16* __restrict__ p_bf16, size_t first,
                                  size_t n, size_t decay_end, float lr, float b1, float b2, float eps, float wd,
                                  float bc1, float bc2, const float* __restrict__ grad_sumsq, float max_grad_norm,
                                  float grad_scale, int mode) {
  const size_t i = first + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float scale;
  if (!optim_clip_scale(grad_sumsq, max_grad_norm, grad_scale, scale)) return;
  const float g = ld_as_float<G>(grad, i) * scale;
  float pi = p[i], mi = m[i], vi = (mode == 2) ? 0.f : v[i];
  optim_update_one(pi, mi, vi, g, (i < decay_end) ? wd : 0.f, lr, b1, b2, eps, bc1, bc2, mode);
  m[i] = mi;
  if (mode != 2) v[i] = vi;
  p[i] = pi;
  if (p_bf16) p_bf16[i] = __float2bfloat16_rn(pi);
}

// Four elements per thread with 16-byte accesses (the update streams 28 bytes per parameter, so it is
// bound by memory bandwidth); covers [0, n4 * 4), 16-byte aligned buffers.
template <typename G>
__global__ void optim_step_vec4_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                       const G* __restrict__ grad, __nv_bfloat16* __restrict__ p_bf16, size_t n4,
                                       size_t decay_end, float lr, float b1, float b2, float eps, float wd,
                                       float bc1, float bc2, const float* __restrict__ grad_sumsq,
                                       float max_grad_norm, float grad_scale, int mode) {
  const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= n4) return;
  float scale;
  if (!optim_clip_scale(grad_sumsq, max_grad_norm, grad_scale, scale)) return;
  const size_t i = t * 4;
  float4 pv = *reinterpret_cast<const float4*>(p + i);
  float4 mv = *reinterpret_cast<const float4*>(m + i);
  float4 vv = (mode == 2) ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(v + i);
  float g[4];
  if constexpr (sizeof(G) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2*>(grad + i);
    g[0] = __uint_as_float(raw.x << 16); g[1] = __uint_as_float(raw.x & 0xffff0000u);
    g[2] = __uint_as_float(raw.y << 16); g[3] = __uint_as_float(raw.y & 0xffff0000u);
  } else {
    const float4 raw = *reinterpret_cast<const float4*>(grad + i);
    g[0] = raw.x; g[1] = raw.y; g[2] = raw.z; g[3] = raw.w;
  }
  float* pp = &pv.x; float* mm = &mv.x; float* vp = &vv.x;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    optim_update_one(pp[j], mm[j], vp[j], g[j] * scale, (i + j < decay_end) ? wd : 0.f, lr, b1, b2, eps, bc1, bc2, mode);
  *reinterpret_cast<float4*>(m + i) = mv;
  if (mode != 2) *reinterpret_cast<float4*>(v + i) = vv;
  *reinterpret_cast<float4*>(p + i) = pv;
  if (p_bf16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(pv.x, pv.y), hi = __floats2bfloat162_rn(pv.z, pv.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p_bf16 + i) = o;
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n,
                                        float scale) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(in[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n,
                                        float scale) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]) * scale;
}

}  // namespace sb

using namespace sb;
#define STREAM static_cast<cudaStream_t>(stream)
#define CHECK_LAUNCH() return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH
static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int sb_rmsnorm_fwd(const void* x, const void* w, void* y, float* inv_rms, int rows, int cols, int ldx,
                              int ldy, float eps, void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || (ldx & 7) || (ldy & 7)) return SB_ERR_ARG;
  if (!al16(x) || !al16(w) || !al16(y)) return SB_ERR_ALIGN;
  const int wpb = 4;
  rmsnorm_fwd_kernel<<<(rows + wpb - 1) / wpb, wpb * 32, 0, STREAM>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
      inv_rms, rows, cols, ldx, ldy, eps);
  CHECK_LAUNCH();
}

// dw_partial: fp32 workspace of ceil(rows/rows_per_chunk)*cols floats; rows_per_chunk
// is fixed at 256 so the summation tree depends only on (rows, cols). (A variant that produced dx and
// the gain-gradient partials in one pass was measured slower: 83 + 20 us against 26 + 23 + 8 us at
// 16384 x 1024, because its register footprint allowed one CTA per SM.)
extern "C" int sb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* inv_rms, const void* dres,
                              void* dx, float* dw_partial, float* dw_f32, void* dw_bf16, int rows, int cols,
                              void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7)) return SB_ERR_ARG;
  if (!al16(dy) || !al16(x) || !al16(w) || !al16(dx) || (dres && !al16(dres))) return SB_ERR_ALIGN;
  const int wpb = 4;
  const dim3 dgrid((rows + wpb - 1) / wpb);
  const __nv_bfloat16 *pdy = static_cast<const __nv_bfloat16*>(dy), *px = static_cast<const __nv_bfloat16*>(x),
                      *pw = static_cast<const __nv_bfloat16*>(w), *pres = static_cast<const __nv_bfloat16*>(dres);
  __nv_bfloat16* pdx = static_cast<__nv_bfloat16*>(dx);
  if (cols == 1024) rmsnorm_bwd_dx_reg_kernel<4><<<dgrid, wpb * 32, 0, STREAM>>>(pdy, px, pw, inv_rms, pres, pdx, rows);
  else if (cols == 2048) rmsnorm_bwd_dx_reg_kernel<8><<<dgrid, wpb * 32, 0, STREAM>>>(pdy, px, pw, inv_rms, pres, pdx, rows);
  else if (cols == 512) rmsnorm_bwd_dx_reg_kernel<2><<<dgrid, wpb * 32, 0, STREAM>>>(pdy, px, pw, inv_rms, pres, pdx, rows);
  else rmsnorm_bwd_dx_kernel<<<dgrid, wpb * 32, 0, STREAM>>>(pdy, px, pw, inv_rms, pres, pdx, rows, cols);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  if (dw_partial) {
    const int rpc = 256;
    const int chunks = (rows + rpc - 1) / rpc;
    dim3 grid((cols + 255) / 256, chunks);
    rmsnorm_bwd_dw_partial_kernel<<<grid, 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(dy),
                                                            static_cast<const __nv_bfloat16*>(x), inv_rms,
                                                            dw_partial, rows, cols, rpc);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
    colsum_finish_kernel<<<(cols + 255) / 256, 256, 0, STREAM>>>(dw_partial, chunks, cols, dw_f32,
                                                                 static_cast<__nv_bfloat16*>(dw_bf16));
  }
  CHECK_LAUNCH();
}

extern "C" int sb_rope(void* x, int ld, int rows, int n_heads, int dh, int seq_len, int offset,
                       const int* positions, const float* cos_t, const float* sin_t, int backward, void* stream) {
  if (rows <= 0 || n_heads <= 0 || (dh & 7) || (ld & 7) || seq_len <= 0) return SB_ERR_ARG;
  if (!al16(x) || !al16(cos_t) || !al16(sin_t)) return SB_ERR_ALIGN;
  const size_t total = static_cast<size_t>(rows) * n_heads * (dh >> 3);
  rope_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, STREAM>>>(
      static_cast<__nv_bfloat16*>(x), ld, rows, n_heads, dh, seq_len, offset, positions, cos_t, sin_t,
      backward ? -1.f : 1.f);
  CHECK_LAUNCH();
}

extern "C" int sb_swiglu_fwd(const void* gu, void* h, int rows, int ff, void* stream) {
  if (rows <= 0 || (ff & 7) || !al16(gu) || !al16(h)) return SB_ERR_ARG;
  const size_t total = static_cast<size_t>(rows) * (ff >> 3);
  swiglu_fwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, STREAM>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), rows, ff);
  CHECK_LAUNCH();
}
extern "C" int sb_swiglu_bwd(const void* gu, const void* dh, void* dgu, int rows, int ff, void* stream) {
  if (rows <= 0 || (ff & 7) || !al16(gu) || !al16(dh) || !al16(dgu)) return SB_ERR_ARG;
  const size_t total = static_cast<size_t>(rows) * (ff >> 3);
  swiglu_bwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, STREAM>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh),
      static_cast<__nv_bfloat16*>(dgu), rows, ff);
  CHECK_LAUNCH();
}
extern "C" int sb_add_bf16(const void* a, const void* b, void* out, size_t n, void* stream) {
  if ((n & 7) || !al16(a) || !al16(b) || !al16(out)) return SB_ERR_ARG;
  const size_t n8 = n >> 3;
  add_bf16_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, STREAM>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(out),
      n8);
  CHECK_LAUNCH();
}

extern "C" int sb_embed_fwd(const void* table, const int64_t* tokens, void* out, int n, int d, int vocab,
                            void* stream) {
  if (n <= 0 || (d & 7) || !al16(table) || !al16(out)) return SB_ERR_ARG;
  embed_fwd_kernel<<<n, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(table), tokens,
                                          static_cast<__nv_bfloat16*>(out), n, d, vocab);
  CHECK_LAUNCH();
}
extern "C" int sb_embed_bwd(const void* dy, const int64_t* sorted_tok, const int64_t* perm, void* dtable, int n,
                            int d, int vocab, int accumulate, void* stream) {
  if (n <= 0 || (d & 7) || !al16(dy) || !al16(dtable)) return SB_ERR_ARG;
  embed_bwd_kernel<<<n, 128, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(dy), sorted_tok, perm,
                                          static_cast<__nv_bfloat16*>(dtable), n, d, vocab, accumulate);
  CHECK_LAUNCH();
}

extern "C" int sb_ce_fwd_bwd(const void* logits, const int64_t* targets, float* loss_rows, void* dlogits, int rows,
                             int cols, int ld, float grad_scale, void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || (ld & 7) || !al16(logits) || (dlogits && !al16(dlogits)))
    return SB_ERR_ARG;
  ce_fwd_bwd_kernel<512><<<rows, 512, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(logits), targets, loss_rows,
                                                   static_cast<__nv_bfloat16*>(dlogits), rows, cols, ld,
                                                   grad_scale);
  CHECK_LAUNCH();
}

// stats: fp32 [rows, 3] = (max, sum exp(x - max), target logit or 0) of the shard starting at vocabulary id v0.
extern "C" int sb_ce_shard_stats(const void* logits, const int64_t* targets, float* stats, int rows, int cols, int ld,
                                 int v0, void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || (ld & 7) || !al16(logits)) return SB_ERR_ARG;
  ce_shard_stats_kernel<512><<<rows, 512, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(logits), targets, stats, rows,
                                                       cols, ld, v0);
  CHECK_LAUNCH();
}
// dlogits (may alias logits) = (exp(x - lse[row]) - onehot) * grad_scale for the shard's columns.
extern "C" int sb_ce_shard_grad(const void* logits, const int64_t* targets, const float* lse, void* dlogits, int rows,
                                int cols, int ld, int v0, float grad_scale, void* stream) {
  if (rows <= 0 || cols <= 0 || (cols & 7) || (ld & 7) || !al16(logits) || !al16(dlogits)) return SB_ERR_ARG;
  ce_shard_grad_kernel<<<rows, 512, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(logits), targets, lse,
                                                 static_cast<__nv_bfloat16*>(dlogits), rows, cols, ld, v0, grad_scale);
  CHECK_LAUNCH();
}

// partials: fp32 workspace of ceil(n/4096) floats.
extern "C" int sb_sumsq(const void* g, size_t n, int is_bf16, float* partials, float* out, int accumulate,
                        void* stream) {
  if (n == 0) return SB_ERR_ARG;
  const size_t nb = (n + kSumsqElemsPerPartial - 1) / kSumsqElemsPerPartial;
  if (nb > 0x7fffffff) return SB_ERR_TOO_LARGE;
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<static_cast<unsigned>(nb), 256, 0, STREAM>>>(
        static_cast<const __nv_bfloat16*>(g), n, partials);
  else
    sumsq_partial_kernel<float><<<static_cast<unsigned>(nb), 256, 0, STREAM>>>(static_cast<const float*>(g), n,
                                                                               partials);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  sumsq_finish_kernel<<<1, 256, 0, STREAM>>>(partials, static_cast<int>(nb), out, accumulate);
  CHECK_LAUNCH();
}

extern "C" int sb_optim_step(float* p, float* m, float* v, const void* grad, int grad_is_bf16, void* p_bf16,
                             size_t n, size_t decay_end, float lr, float b1, float b2, float eps, float wd,
                             float bc1, float bc2, const float* grad_sumsq, float max_grad_norm, float grad_scale,
                             int mode, void* stream) {
  if (n == 0) return SB_ERR_ARG;
  const bool aligned = al16(p) && al16(m) && (mode == 2 || al16(v)) && al16(grad) &&
                       (!p_bf16 || (reinterpret_cast<uintptr_t>(p_bf16) & 7) == 0);
  const size_t n4 = aligned ? n / 4 : 0;
  const size_t first = n4 * 4;
  if (n4) {
    const unsigned blocks = static_cast<unsigned>((n4 + 255) / 256);
    if (grad_is_bf16)
      optim_step_vec4_kernel<__nv_bfloat16><<<blocks, 256, 0, STREAM>>>(
          p, m, v, static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(p_bf16), n4, decay_end, lr,
          b1, b2, eps, wd, bc1, bc2, grad_sumsq, max_grad_norm, grad_scale, mode);
    else
      optim_step_vec4_kernel<float><<<blocks, 256, 0, STREAM>>>(p, m, v, static_cast<const float*>(grad),
                                                                static_cast<__nv_bfloat16*>(p_bf16), n4, decay_end,
                                                                lr, b1, b2, eps, wd, bc1, bc2, grad_sumsq,
                                                                max_grad_norm, grad_scale, mode);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  if (first < n) {
    const unsigned blocks = static_cast<unsigned>((n - first + 255) / 256);
    if (grad_is_bf16)
      optim_step_kernel<__nv_bfloat16><<<blocks, 256, 0, STREAM>>>(
          p, m, v, static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(p_bf16), first, n, decay_end,
          lr, b1, b2, eps, wd, bc1, bc2, grad_sumsq, max_grad_norm, grad_scale, mode);
    else
      optim_step_kernel<float><<<blocks, 256, 0, STREAM>>>(p, m, v, static_cast<const float*>(grad),
                                                           static_cast<__nv_bfloat16*>(p_bf16), first, n, decay_end, lr,
                                                           b1, b2, eps, wd, bc1, bc2, grad_sumsq, max_grad_norm,
                                                           grad_scale, mode);
  }
  CHECK_LAUNCH();
}

extern "C" int sb_cast(const void* in, void* out, size_t n, int to_bf16, float scale, void* stream) {
  if (n == 0) return SB_ERR_ARG;
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  if (to_bf16)
    cast_f32_to_bf16_kernel<<<blocks, 256, 0, STREAM>>>(static_cast<const float*>(in),
                                                        static_cast<__nv_bfloat16*>(out), n, scale);
  else
    cast_bf16_to_f32_kernel<<<blocks, 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(in),
                                                        static_cast<float*>(out), n, scale);
  CHECK_LAUNCH();
}

// Multi-tensor cast: up to MULTI_CAST_MAX fp32 tensors are rounded to bf16 into slices of one flat
// buffer in a single launch (a data-parallel bucket's gradients). blockIdx.y selects the tensor.
constexpr int MULTI_CAST_MAX = 96;
struct MultiCastParams {
  const float* src[MULTI_CAST_MAX];
  unsigned long long dst_off[MULTI_CAST_MAX];   // element offset into dst
  unsigned long long n[MULTI_CAST_MAX];
};
__global__ void multi_cast_f32_bf16_kernel(const __grid_constant__ MultiCastParams p, __nv_bfloat16* __restrict__ dst,
                                           int accumulate) {
  const int t = blockIdx.y;
  const float* __restrict__ s = p.src[t];
  __nv_bfloat16* __restrict__ d = dst + p.dst_off[t];
  const size_t n = p.n[t];
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float v = s[i];
    if (accumulate) v += __bfloat162float(d[i]);
    d[i] = __float2bfloat16_rn(v);
  }
}

// srcs / dst_offs / ns: host arrays of `count` entries (count <= 96). dst: bf16 flat buffer.
extern "C" int sb_multi_cast_f32_bf16(const void* const* srcs, const unsigned long long* dst_offs,
                                      const unsigned long long* ns, int count, void* dst, int accumulate,
                                      void* stream) {
  if (count < 1 || count > MULTI_CAST_MAX || dst == nullptr) return SB_ERR_ARG;
  MultiCastParams p;
  unsigned long long nmax = 0;
  for (int i = 0; i < count; ++i) {
    if (srcs[i] == nullptr) return SB_ERR_ARG;
    p.src[i] = static_cast<const float*>(srcs[i]);
    p.dst_off[i] = dst_offs[i];
    p.n[i] = ns[i];
    if (ns[i] > nmax) nmax = ns[i];
  }
  if (nmax == 0) return SB_ERR_ARG;
  unsigned bx = static_cast<unsigned>((nmax + 255) / 256);
  if (bx > 1024) bx = 1024;
  multi_cast_f32_bf16_kernel<<<dim3(bx, count), 256, 0, STREAM>>>(p, static_cast<__nv_bfloat16*>(dst), accumulate);
  CHECK_LAUNCH();
}

// ---------------------------------------------------------------------------
// sb_sumsq_no_alloc: the sum of squares for callers that cannot allocate (see
// sumsq_no_alloc.h). Same kernels and launch shape as sb_sumsq; the per-block partials go to
// an array that is part of the library image instead of a caller-provided buffer.
// ---------------------------------------------------------------------------
#include "sumsq_no_alloc.h"
static_assert(SB_SUMSQ_NO_ALLOC_ELEMS_PER_PARTIAL == kSumsqElemsPerPartial,
              "the header's limit must describe the partial size the kernels use");

static __device__ __align__(256) float g_sumsq_no_alloc_scratch[SB_SUMSQ_NO_ALLOC_MAX_PARTIALS];

// Device address of the scratch array, resolved once per device. In host code the array's name
// is only a handle for the runtime, not something a kernel can dereference.
static float* g_sumsq_no_alloc_ptr[64] = {nullptr};

extern "C" int sb_sumsq_no_alloc(const void* g, size_t n, int is_bf16, float* out, int accumulate, void* stream) {
  if (n == 0 || g == nullptr || out == nullptr) return SB_ERR_ARG;
  if (n > SB_SUMSQ_NO_ALLOC_MAX_ELEMS) return SB_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SB_ERR_RUNTIME;
  float* scratch = g_sumsq_no_alloc_ptr[dev];
  if (scratch == nullptr) {
    // first call on this device (which is current): ask the runtime where the array lives here
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sumsq_no_alloc_scratch) != cudaSuccess || p == nullptr) return SB_ERR_RUNTIME;
    scratch = static_cast<float*>(p);
    g_sumsq_no_alloc_ptr[dev] = scratch;
  }
  const size_t nb = (n + kSumsqElemsPerPartial - 1) / kSumsqElemsPerPartial;
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<static_cast<unsigned>(nb), 256, 0, STREAM>>>(
        static_cast<const __nv_bfloat16*>(g), n, scratch);
  else
    sumsq_partial_kernel<float><<<static_cast<unsigned>(nb), 256, 0, STREAM>>>(static_cast<const float*>(g), n,
                                                                               scratch);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  sumsq_finish_kernel<<<1, 256, 0, STREAM>>>(scratch, static_cast<int>(nb), out, accumulate);
  CHECK_LAUNCH();
}
