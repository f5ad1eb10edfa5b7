// Work scheduling shared by the persistent GEMM kernels.
//
// "Balanced" schedule: the first dp_tiles output tiles (whole waves of the grid) are processed one
// tile per worker visit; the k-blocks of the remaining sk_tiles tiles (the last, partial wave) are
// dealt out evenly to the first sk_workers workers. A worker may therefore hold only a PART of a
// tile: such a part is written as a dense fp32 block to a scratch slot and balanced_fixup_kernel adds
// the parts of a tile in ascending k (= ascending worker index), so the summation order is a function
// of the shape and the grid only. A worker is a CTA, or a CTA pair for the cta_group::2 kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb {

struct BalancedSched {
  int dp_tiles, sk_tiles, sk_workers, sk_slots;   // sk_tiles == 0: plain one-tile-per-visit schedule
};

// One unit of work: k-blocks [kb0, kb1) of tile `tile` (split-K index `split` for the explicit
// split-K mode); slot < 0 means the result is final and goes to C.
struct Seg {
  int tile, split, kb0, kb1, slot;
};

struct SegIter {
  BalancedSched s;
  int worker, n_workers, tiles_mn, num_kb, splits, kb_per_split;
  int t;
  long long u, u_hi;
  int ordinal;
  __device__ SegIter(const BalancedSched& s_, int worker_, int n_workers_, int tiles_mn_, int num_kb_, int splits_,
                     int kb_per_split_)
      : s(s_), worker(worker_), n_workers(n_workers_), tiles_mn(tiles_mn_), num_kb(num_kb_), splits(splits_),
        kb_per_split(kb_per_split_), t(worker_), u(0), u_hi(0), ordinal(0) {
    if (s.sk_tiles > 0 && worker < s.sk_workers) {
      const long long U = static_cast<long long>(s.sk_tiles) * num_kb;
      u = U * worker / s.sk_workers;
      u_hi = U * (worker + 1) / s.sk_workers;
    }
  }
  __device__ bool next(Seg& g) {
    const int dp_total = s.sk_tiles > 0 ? s.dp_tiles : tiles_mn * splits;
    if (t < dp_total) {
      g.split = t / tiles_mn;
      g.tile = t - g.split * tiles_mn;
      g.kb0 = g.split * kb_per_split;
      g.kb1 = min(num_kb, g.kb0 + kb_per_split);
      g.slot = -1;
      t += n_workers;
      return true;
    }
    if (u < u_hi) {
      const int r = static_cast<int>(u / num_kb);
      g.split = 0;
      g.tile = s.dp_tiles + r;
      g.kb0 = static_cast<int>(u - static_cast<long long>(r) * num_kb);
      g.kb1 = static_cast<int>(min(static_cast<long long>(num_kb), g.kb0 + (u_hi - u)));
      g.slot = (g.kb0 == 0 && g.kb1 == num_kb) ? -1 : worker * s.sk_slots + ordinal;
      ++ordinal;
      u += g.kb1 - g.kb0;
      return true;
    }
    return false;
  }
};

// Host: plan the schedule for `tiles` tiles of `num_kb` k-blocks on `workers` workers. Returns false
// (plain schedule) when every tile belongs to a whole wave. *fixup tells whether any tile is split.
inline bool plan_balanced(int tiles, int num_kb, int workers, BalancedSched* out, bool* fixup) {
  out->dp_tiles = out->sk_tiles = out->sk_workers = out->sk_slots = 0;
  *fixup = false;
  const int dp = (tiles / workers) * workers, sk = tiles - dp;
  if (sk == 0) return false;
  const long long U = static_cast<long long>(sk) * num_kb;
  long long w = U / 4;                     // at least four k-blocks per part
  if (w < 1) w = 1;
  if (w > workers) w = workers;
  if (w < sk) w = sk;                      // never fewer workers than tiles (sk < workers)
  const int slots = static_cast<int>(((U / w + 1) + num_kb - 1) / num_kb) + 1;
  if (slots > 3) return false;
  out->dp_tiles = dp;
  out->sk_tiles = sk;
  out->sk_workers = static_cast<int>(w);
  out->sk_slots = slots;
  for (long long c = 1; c < w && !*fixup; ++c) *fixup = (U * c / w) % num_kb != 0;
  return true;
}

__device__ __forceinline__ float sched_bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float sched_bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Finishes the split tiles. Tile = TM x TN outputs, parts are dense fp32 [TM, TN] blocks at
// partials + slot * TM * TN. grid = (sk_tiles, TM * TN / (256 * 4)), 256 threads.
template <int TM, int TN>
__global__ void balanced_fixup_kernel(BalancedSched s, const float* __restrict__ partials, __nv_bfloat16* __restrict__ C,
                                      int ldc, const __nv_bfloat16* __restrict__ R, int ldr, int M, int N, int mt,
                                      int num_kb) {
  const int r = blockIdx.x;
  const long long U = static_cast<long long>(s.sk_tiles) * num_kb;
  const long long lo = static_cast<long long>(r) * num_kb, hi = lo + num_kb;
  int c = static_cast<int>(lo * s.sk_workers / U);
  while (c > 0 && U * c / s.sk_workers > lo) --c;
  while (U * (c + 1) / s.sk_workers <= lo) ++c;
  {
    const long long u0 = U * c / s.sk_workers, u1 = U * (c + 1) / s.sk_workers;
    if (u0 <= lo && u1 >= hi) return;   // computed whole by one worker
  }
  const int tile = s.dp_tiles + r;
  const int n_idx = tile / mt, m_idx = tile - n_idx * mt;
  const int e = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const int tr = e / TN, tc = e - tr * TN;
  const int row = m_idx * TM + tr, col = n_idx * TN + tc;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  // the parts of this tile, in ascending k (= ascending worker); eight loads are in flight before the first add and
  // the adds keep the part order, so the sum is the same whatever the grouping
  while (c < s.sk_workers) {
    const float* src[8];
    int n = 0;
    for (; c < s.sk_workers && n < 8; ++c) {
      const long long u0 = U * c / s.sk_workers, u1 = U * (c + 1) / s.sk_workers;
      if (u0 >= hi) { c = s.sk_workers; break; }
      if (u1 <= lo || u1 == u0) continue;
      const int ordinal = r - static_cast<int>(u0 / num_kb);
      const size_t slot = static_cast<size_t>(c) * s.sk_slots + ordinal;
      src[n++] = partials + (slot * TM + tr) * TN + tc;
    }
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < n) v[i] = __ldcs(reinterpret_cast<const float4*>(src[i]));
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < n) { acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w; }
  }
  if (row >= M || col >= N) return;
  if (R) {
    const uint2 rv = *reinterpret_cast<const uint2*>(R + static_cast<size_t>(row) * ldr + col);
    acc.x += sched_bf16_lo(rv.x); acc.y += sched_bf16_hi(rv.x);
    acc.z += sched_bf16_lo(rv.y); acc.w += sched_bf16_hi(rv.y);
  }
  __nv_bfloat162 o0 = __floats2bfloat162_rn(acc.x, acc.y), o1 = __floats2bfloat162_rn(acc.z, acc.w);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&o0);
  o.y = *reinterpret_cast<uint32_t*>(&o1);
  *reinterpret_cast<uint2*>(C + static_cast<size_t>(row) * ldc + col) = o;
}

}  // namespace sb
