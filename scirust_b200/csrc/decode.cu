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
#include <cuda_fp16.h>
#include <cstdlib>
#include "sm100_ptx.cuh"
#include "peer_sync.cuh"

namespace sb {

__device__ __forceinline__ float dbflo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float dbfhi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t dpack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start
// while its predecessor in the stream is still draining. Work that does not depend on the
// predecessor (weight prefetch, barrier set-up) runs at once; pdl_wait() returns when the predecessor
// has completed and its writes are visible, and must precede every read of its results and every
// global write. pdl_trigger() tells the scheduler that this CTA no longer minds dependents being
// co-scheduled. Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------
// GEMV / skinny GEMM: Y[M,N] = f(X)[M,K] * W[K,N] (* scale[n]) (+ R), M <= MB <= 8, W streamed once.
// grid = (ceil(N / COLS), splits). A CTA owns COLS output columns (512 bytes of every weight row)
// and the k range of its split.
//   warp 8      producer: streams the CTA's weight slab through a ring of STAGES tiles of 32 rows,
//               one 16 KB TMA tile copy and one mbarrier per stage (copies of single 512-byte rows
//               reached less than half of the memory bandwidth); it starts at once, because the
//               weights do not depend on the previous kernel's output
//   warps 0-7   stage f(X) for the CTA's k range in shared memory (optionally fused RMSNorm or
//               SwiGLU), then consume tiles: warp w takes rows w, w+8, w+16, w+24 of every tile, a
//               lane holds VEC consecutive columns
// Partials of the 8 warps are added in warp order in shared memory; split partials go to a
// workspace and the LAST CTA of a column block (a counter, no data atomics) adds them in split
// order and applies scale / residual: the summation tree depends only on (K, splits), and the
// finishing pass needs no second launch.
// INT8: W is int8 with one fp32 scale per output column, applied after the sum.
// ---------------------------------------------------------------------------
constexpr int GEMV_KT = 32;          // rows per tile
constexpr int GEMV_ROW_BYTES = 512;  // bytes of one weight row owned by a CTA
constexpr int GEMV_STAGES = 4;   // 64 KB ring: three CTAs fit on an SM, so a dependent kernel's CTAs
                                 // find room to prefetch their weights while this kernel still runs
constexpr int GEMV_TILE_BYTES = GEMV_KT * GEMV_ROW_BYTES;
constexpr int GEMV_THREADS = 288;
constexpr int GEMV_MAX_XS_BYTES = 64 * 1024;

// Optional prologue applied to X while it is staged (so the producing kernel disappears):
//   PRO_RMSNORM: x <- bf16(x * rsqrt(mean(x^2) + eps) * norm_w[k]); the row statistic is computed by
//                one warp per row in exactly the order of rmsnorm_fwd_kernel, so fused and unfused
//                paths agree bit for bit.
//   PRO_SWIGLU:  X is a fused [gate | up] row of width 2K: x <- bf16(silu(gate[k]) * up[k]).
enum { PRO_NONE = 0, PRO_RMSNORM = 1, PRO_SWIGLU = 2 };

struct GemvParams {
  const __nv_bfloat16* X; int ldx;
  const void* W; int ldw;            // elements
  const float* scale;                // int8 only
  const __nv_bfloat16* R; int ldr;
  __nv_bfloat16* out; int ldo;
  float* out_f32;                    // [M, N] dense, optional
  float* part;                       // [splits, M, N] when splits > 1
  unsigned int* counters;            // [gridDim.x], zero between calls
  int M, N, K, k_per_split, prologue;
  const __nv_bfloat16* norm_w; float eps;
  int* status;
  // Row-parallel product fused with its all-reduce (coll.W > 1; tensor-parallel decoding): the CTA that finishes a
  // block of output columns does not write its rank's partial sums to local memory for a second kernel to combine;
  // it stores them (fp32, before the residual) into slot [parity][rank] of EVERY rank's receive buffer with plain
  // peer stores, raises the column block's flag on every rank, waits (bounded) for the W flags of its own column
  // block and adds the W slots in rank order on top of the residual. Every rank adds the same values in the same
  // order, so all ranks hold identical bits, the same bits as the GEMV followed by the stand-alone all-reduce.
  //   recv[r]   rank r's receive buffer, fp32 [2][W][coll.rows][N]; a call uses half `epoch & 1`, so a rank that is
  //             one call ahead never overwrites what a slower rank is still adding
  //   flags[r]  rank r's epoch words [column block][MAX_WORLD]
  //   epoch_word / done_ctr: local words; the call's epoch is *epoch_word + 1 and the last finishing CTA stores it
  //             back, so a captured CUDA graph replays the call with the right epoch.
  struct {
    int W, rank, rows;
    float* recv[MAX_WORLD];
    uint32_t* flags[MAX_WORLD];
    uint32_t* epoch_word;
    unsigned int* done_ctr;
    uint64_t wait_ns;
  } coll;
  // LM head fused with the greedy arg-max (amax.out_tokens != nullptr; scirust-cuda/src/bf16_lm_head_argmax.rs:46-176):
  // the CTA that finishes a block of columns keeps its final values in shared memory, reduces them to one
  // (value, column) per row and the last CTA of the grid reduces those and writes the token to the device-side
  // feedback buffer: no logits round trip, no second and third launch. With amax.W > 1 the head is sharded over
  // the vocabulary (col_offset = first global column of this rank): the last CTA stores the rank's candidates into
  // slot [parity][rank] of every rank's `cand`, raises its flag on every rank, waits (bounded) for the W flags and
  // reduces the W candidates, so every rank writes the same token.
  struct {
    float* pval; int* pidx;            // [M][gridDim.x]
    unsigned int* ctr;                 // zero between calls
    int64_t* out_tokens; int64_t* generated; int gen_stride, step;
    int col_offset, W, rank;
    unsigned long long* cand[MAX_WORLD];   // rank r's candidates: [2][W][8] of (value bits << 32 | column)
    uint32_t* flags[MAX_WORLD];            // rank r's epoch words [MAX_WORLD]
    uint32_t* epoch_word;
    uint64_t wait_ns;
  } amax;
};

// Arg-max order of the greedy loop (`best = row[0]; if v > best`, scirust-cuda/src/decode.rs:107-114): the larger
// value wins, among equal values the lower column. Both operands are numbers (NaN never enters); -inf at a real
// column beats the empty sentinel (-inf, 0x7fffffff).
__device__ __forceinline__ bool argmax_better(float v, int i, float best, int bi) {
  return v > best || (v == best && i < bi);
}
__device__ __forceinline__ void warp_argmax(float& best, int& bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
  }
}

// Tail of the fused LM head: `vals[m * cols_per_cta + c]` holds the final values of this CTA's `ncols` columns.
__device__ __noinline__ void gemv_argmax_tail(const GemvParams& p, float* vals, int cols_per_cta, int col0, int ncols,
                                              int* s_flag) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int nblk = gridDim.x;
  constexpr int NONE = 0x7fffffff;
  __syncthreads();
  for (int m = warp; m < p.M; m += nw) {
    float best = -INFINITY;
    int bi = NONE;
    for (int c = lane; c < ncols; c += 32) {
      const float v = vals[m * cols_per_cta + c];
      if (v != v) continue;                        // a NaN is skipped explicitly ...
      const int gi = p.amax.col_offset + col0 + c;
      if (argmax_better(v, gi, best, bi)) { best = v; bi = gi; }
    }
    warp_argmax(best, bi);
    if (lane == 0) {
      if (col0 == 0 && p.amax.col_offset == 0) {   // ... except in column 0, where it makes token 0 win outright
        const float f = vals[m * cols_per_cta];
        if (f != f) { best = INFINITY; bi = 0; }
      }
      p.amax.pval[m * nblk + blockIdx.x] = best;
      p.amax.pidx[m * nblk + blockIdx.x] = bi;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.amax.ctr, 1u);
    *s_flag = (prev == static_cast<unsigned int>(nblk) - 1u) ? 1 : 0;
    if (*s_flag) *p.amax.ctr = 0;
  }
  __syncthreads();
  if (!*s_flag) return;
  __threadfence();
  const int W = p.amax.W;
  const uint32_t epoch = W > 1 ? *reinterpret_cast<volatile uint32_t*>(p.amax.epoch_word) + 1u : 0u;
  for (int m = warp; m < p.M; m += nw) {
    float best = -INFINITY;
    int bi = NONE;
    for (int s = lane; s < nblk; s += 32) {
      const float v = __ldcg(p.amax.pval + m * nblk + s);
      const int i = __ldcg(p.amax.pidx + m * nblk + s);
      if (argmax_better(v, i, best, bi)) { best = v; bi = i; }
    }
    warp_argmax(best, bi);
    if (W <= 1) {
      if (lane == 0) {
        if (bi == NONE) bi = 0;                    // no number in the row
        p.amax.out_tokens[m] = bi;
        if (p.amax.generated) p.amax.generated[static_cast<size_t>(m) * p.amax.gen_stride + p.amax.step] = bi;
      }
    } else if (lane < W) {
      const unsigned long long pk = (static_cast<unsigned long long>(__float_as_uint(best)) << 32) |
                                    static_cast<uint32_t>(bi);
      p.amax.cand[lane][(static_cast<size_t>(epoch & 1u) * W + p.amax.rank) * 8 + m] = pk;
    }
  }
  if (W <= 1) return;
  __syncthreads();          // every candidate store is ordered before the fence of the announcing lanes
  if (threadIdx.x < 32) {
    if (static_cast<int>(threadIdx.x) < W) {
      __threadfence_system();
      st_release_sys(p.amax.flags[threadIdx.x] + p.amax.rank, epoch);
    }
    const bool ok = wait_flags_warp(p.amax.flags[p.amax.rank], W, epoch, p.amax.wait_ns, p.status);
    if (threadIdx.x == 0) *s_flag = ok ? 1 : 0;
  }
  __syncthreads();
  if (*s_flag) {
    for (int m = warp; m < p.M; m += nw) {
      float best = -INFINITY;
      int bi = NONE;
      if (lane < W) {
        const unsigned long long pk = __ldcg(p.amax.cand[p.amax.rank] + (static_cast<size_t>(epoch & 1u) * W + lane) * 8 + m);
        best = __uint_as_float(static_cast<uint32_t>(pk >> 32));
        bi = static_cast<int>(static_cast<uint32_t>(pk));
      }
      warp_argmax(best, bi);
      if (lane == 0) {
        if (bi == NONE) bi = 0;
        p.amax.out_tokens[m] = bi;
        if (p.amax.generated) p.amax.generated[static_cast<size_t>(m) * p.amax.gen_stride + p.amax.step] = bi;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(p.amax.epoch_word) = epoch;
}

// One finished partial sum (m, gc) of the fused all-reduce path: to slot [parity][rank] of every rank.
__device__ __forceinline__ void gemv_coll_push(const GemvParams& p, uint32_t epoch, int m, int gc, float sum) {
  const size_t off = ((static_cast<size_t>(epoch & 1u) * p.coll.W + p.coll.rank) * p.coll.rows + m) * p.N + gc;
  for (int r = 0; r < p.coll.W; ++r) p.coll.recv[(p.coll.rank + r) % p.coll.W][off] = sum;
}

// Tail of the fused all-reduce path, called by all threads of the CTA that finished column block blockIdx.x.
__device__ __forceinline__ void gemv_coll_finish(const GemvParams& p, uint32_t epoch, int col0, int ncols, int* s_flag) {
  const int W = p.coll.W;
  __syncthreads();      // every thread's pushes are ordered before the fence of the announcing lanes (cumulative release)
  if (threadIdx.x < 32) {
    if (static_cast<int>(threadIdx.x) < W) {
      __threadfence_system();
      st_release_sys(p.coll.flags[threadIdx.x] + blockIdx.x * MAX_WORLD + p.coll.rank, epoch);
    }
    const bool ok = wait_flags_warp(p.coll.flags[p.coll.rank] + blockIdx.x * MAX_WORLD, W, epoch, p.coll.wait_ns, p.status);
    if (threadIdx.x == 0) *s_flag = ok ? 1 : 0;
  }
  __syncthreads();
  if (*s_flag) {
    const float* mine = p.coll.recv[p.coll.rank] + static_cast<size_t>(epoch & 1u) * W * p.coll.rows * p.N;
    const size_t rstride = static_cast<size_t>(p.coll.rows) * p.N;
    for (int i = threadIdx.x; i < p.M * ncols; i += blockDim.x) {
      const int m = i / ncols, gc = col0 + (i - m * ncols);
      float acc = p.R ? __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]) : 0.f;
      const float* src = mine + static_cast<size_t>(m) * p.N + gc;
      for (int r0 = 0; r0 < W; r0 += 8) {      // eight loads in flight, added in rank order
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = (r0 + u < W) ? __ldcg(src + (r0 + u) * rstride) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) if (r0 + u < W) acc += v[u];
      }
      if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(acc);
      if (p.out_f32) p.out_f32[static_cast<size_t>(m) * p.N + gc] = acc;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(p.coll.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *p.coll.done_ctr = 0;
      *reinterpret_cast<volatile uint32_t*>(p.coll.epoch_word) = epoch;
    }
  }
}

template <int MB, bool INT8>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ GemvParams p) {
  constexpr int VEC = INT8 ? 16 : 8;
  constexpr int COLS = 32 * VEC;
  constexpr int ESZ = INT8 ? 1 : 2;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* tiles = smem;                                                  // STAGES x 16 KB
  float* xs = reinterpret_cast<float*>(smem + GEMV_STAGES * GEMV_TILE_BYTES);  // [k][MB]
  __shared__ uint64_t full[GEMV_STAGES], empty[GEMV_STAGES];
  __shared__ float s_inv[8];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = p.M, N = p.N, K = p.K;
  const int col0 = blockIdx.x * COLS;
  const int k0 = blockIdx.y * p.k_per_split;
  const int k1 = min(K, k0 + p.k_per_split);
  const int ntiles = (k1 - k0 + GEMV_KT - 1) / GEMV_KT;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_w);
    for (int s = 0; s < GEMV_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 8); }
    fence_barrier_init();
  }
  __syncthreads();

  float acc[MB][VEC];
#pragma unroll
  for (int m = 0; m < MB; ++m)
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[m][j] = 0.f;

  if (warp == 8) {
    // ------------------------------ producer ------------------------------
    // the map is over 16-bit words: x = byte offset of the CTA's columns / 2 (a multiple of 256)
    const int x0 = col0 * ESZ / 2;
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % GEMV_STAGES;
      if (t >= GEMV_STAGES && !mbar_wait(&empty[s], ((t / GEMV_STAGES) - 1) & 1, p.status, ST_TIMEOUT_EMPTY)) break;
      if (lane == 0) {
        // rows past K and columns past N arrive as zeros and still count towards the byte total
        mbar_arrive_expect_tx(&full[s], GEMV_TILE_BYTES);
        tma_load_2d(tiles + s * GEMV_TILE_BYTES, &tmap_w, &full[s], x0, k0 + t * GEMV_KT);
      }
      __syncwarp();
    }
    pdl_wait();   // this warp writes results below
  } else {
    // ------------------------------ consumers -----------------------------
    pdl_wait();   // X, the residual and the workspace belong to the previous kernel until here
    if (p.prologue == PRO_RMSNORM) {
      // row statistic with the association of rmsnorm_fwd_kernel: per lane, accumulator a takes the
      // 16-byte chunks lane*8 + 256*(a + 8*j); here warp a computes accumulator a of every row
      float* s_part = xs;   // [M][8 warps][32 lanes], overwritten by the staging below
      if (M == 1) {
        const __nv_bfloat16* xr = p.X;
        float a = 0.f;
        for (int c = lane * 8 + warp * 256; c < K; c += 8 * 256) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
          const float f[8] = {dbflo(raw.x), dbfhi(raw.x), dbflo(raw.y), dbfhi(raw.y),
                              dbflo(raw.z), dbfhi(raw.z), dbflo(raw.w), dbfhi(raw.w)};
#pragma unroll
          for (int j = 0; j < 8; ++j) a += f[j] * f[j];
        }
        s_part[warp * 32 + lane] = a;
      } else {
        // all rows of one column step are loaded before the first use; per row the adds keep their order
        float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int c = lane * 8 + warp * 256; c < K; c += 8 * 256) {
          uint4 raw[8];
#pragma unroll
          for (int m = 0; m < 8; ++m)
            if (m < M) raw[m] = *reinterpret_cast<const uint4*>(p.X + static_cast<size_t>(m) * p.ldx + c);
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            if (m < M) {
              const float f[8] = {dbflo(raw[m].x), dbfhi(raw[m].x), dbflo(raw[m].y), dbfhi(raw[m].y),
                                  dbflo(raw[m].z), dbfhi(raw[m].z), dbflo(raw[m].w), dbfhi(raw[m].w)};
#pragma unroll
              for (int j = 0; j < 8; ++j) a8[m] += f[j] * f[j];
            }
          }
        }
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < M) s_part[(m * 8 + warp) * 32 + lane] = a8[m];
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      for (int m = warp; m < M; m += 8) {
        float ss = s_part[(m * 8) * 32 + lane];
#pragma unroll
        for (int a = 1; a < 8; ++a) ss += s_part[(m * 8 + a) * 32 + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_inv[m] = rsqrtf(ss / static_cast<float>(K) + p.eps);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    const int kn_all = k1 - k0;
    for (int i = threadIdx.x; i < kn_all * MB; i += 256) {
      const int kk = i / MB, m = i - kk * MB;
      float xv = 0.f;
      if (m < M) {
        const int k = k0 + kk;
        xv = __bfloat162float(p.X[static_cast<size_t>(m) * p.ldx + k]);
        if (p.prologue == PRO_RMSNORM) {
          xv = __bfloat162float(__float2bfloat16_rn(xv * s_inv[m] * __bfloat162float(p.norm_w[k])));
        } else if (p.prologue == PRO_SWIGLU) {
          const float u = __bfloat162float(p.X[static_cast<size_t>(m) * p.ldx + K + k]);
          xv = __bfloat162float(__float2bfloat16_rn(xv / (1.f + __expf(-xv)) * u));
        }
      }
      xs[i] = xv;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    const bool active = lane * VEC < min(COLS, N - col0);
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % GEMV_STAGES;
      if (!mbar_wait(&full[s], (t / GEMV_STAGES) & 1, p.status, ST_TIMEOUT_FULL)) break;
      const int rows = min(GEMV_KT, k1 - (k0 + t * GEMV_KT));
      const uint8_t* tile = tiles + s * GEMV_TILE_BYTES;
      uint4 raw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = warp + i * 8;
        raw[i] = (active && r < rows) ? *reinterpret_cast<const uint4*>(tile + r * GEMV_ROW_BYTES + lane * 16)
                                      : make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = warp + i * 8;
        if (r >= rows) continue;
        float w[VEC];
        if constexpr (INT8) {
          // int8 -> fp32 without the slow conversion pipe: flip the sign bit (value + 128 as an
          // unsigned byte), drop the byte into the low mantissa of 2^23 and subtract 2^23 + 128
          const uint32_t words[4] = {raw[i].x ^ 0x80808080u, raw[i].y ^ 0x80808080u, raw[i].z ^ 0x80808080u,
                                     raw[i].w ^ 0x80808080u};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            w[q * 4 + 0] = __uint_as_float(__byte_perm(words[q], 0x4B000000u, 0x7540)) - 8388736.0f;
            w[q * 4 + 1] = __uint_as_float(__byte_perm(words[q], 0x4B000000u, 0x7541)) - 8388736.0f;
            w[q * 4 + 2] = __uint_as_float(__byte_perm(words[q], 0x4B000000u, 0x7542)) - 8388736.0f;
            w[q * 4 + 3] = __uint_as_float(__byte_perm(words[q], 0x4B000000u, 0x7543)) - 8388736.0f;
          }
        } else {
          w[0] = dbflo(raw[i].x); w[1] = dbfhi(raw[i].x); w[2] = dbflo(raw[i].y); w[3] = dbfhi(raw[i].y);
          w[4] = dbflo(raw[i].z); w[5] = dbfhi(raw[i].z); w[6] = dbflo(raw[i].w); w[7] = dbfhi(raw[i].w);
        }
        const float* xr = xs + (t * GEMV_KT + r) * MB;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          const float xv = xr[m];
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[m][j] += xv * w[j];
        }
      }
    }
  }
  // every tile has been consumed (or a wait gave up and no copy is read any more): reuse the ring
  // for the cross-warp reduction, one output row at a time, warps added in warp order
  __syncthreads();
  // the weight stream of this CTA is done: the next kernel in the stream may be co-scheduled, so that
  // its weight prefetch overlaps this kernel's reduction tail. (Triggering at kernel start instead
  // was measured slower: 3.84 against 3.68 ms per Llama-3-8B-shape token without any overlap.)
  pdl_trigger();
  float* buf = reinterpret_cast<float*>(tiles);  // [8 warps][32 lanes][VEC]
  const bool direct = gridDim.y == 1;
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    if (warp < 8) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) buf[(warp * 32 + lane) * VEC + j] = acc[m][j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < COLS; c += GEMV_THREADS) {
      const int l = c / VEC, j = c - l * VEC;
      float sum = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) sum += buf[(w8 * 32 + l) * VEC + j];
      const int gc = col0 + c;
      if (m < M && gc < N) {
        if (direct) {
          if (p.scale) sum *= p.scale[gc];
          if (p.R) sum += __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]);
          if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(sum);
          if (p.out_f32) p.out_f32[static_cast<size_t>(m) * N + gc] = sum;
        } else {
          p.part[(static_cast<size_t>(blockIdx.y) * M + m) * N + gc] = sum;
        }
      }
    }
    __syncthreads();
  }
  if (direct) return;
  // split-K finish by the last CTA of this column block
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.counters + blockIdx.x, 1u);
    s_last = (prev == gridDim.y - 1) ? 1 : 0;
    if (s_last) p.counters[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int ncols = min(COLS, N - col0);
  for (int i = threadIdx.x; i < M * ncols; i += GEMV_THREADS) {
    const int m = i / ncols, gc = col0 + (i - m * ncols);
    float sum = 0.f;
    const float* pp = p.part + static_cast<size_t>(m) * N + gc;
    const size_t pstride = static_cast<size_t>(M) * N;
    const int ns = static_cast<int>(gridDim.y);
    for (int k = 0; k < ns; k += 8) {   // eight loads in flight, added in split order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (k + u < ns) ? __ldcg(pp + (k + u) * pstride) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) if (k + u < ns) sum += v[u];
    }
    if (p.scale) sum *= p.scale[gc];
    if (p.R) sum += __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]);
    if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(sum);
    if (p.out_f32) p.out_f32[static_cast<size_t>(m) * N + gc] = sum;
  }
}

// ---------------------------------------------------------------------------
// bf16 GEMV on tensor cores. The FMA kernel above spends about five thread instructions per weight
// (unpack, convert, multiply-add) and is bound by instruction issue at 0.55-0.7 of the memory
// bandwidth; here a warp turns a 16 (k) x 16 (n) block of weights into one ldmatrix.x4.trans and one
// mma.sync.m16n8k16: the weights are the A operand (W^T: n rows, k columns), the up to 8 activation
// rows are the 8 columns of B (unused columns are zero), and the accumulator holds 16 outputs x 8
// rows in fp32. Same grid, ring, producer warp, prologues and split-K finish as the FMA kernel; the
// weight tile arrives as four 128-byte-swizzled [32 k x 64 n] boxes so that ldmatrix is free of
// bank conflicts; warp w owns columns [32w, 32w+32) of the CTA's 256, so no cross-warp sum exists.
// The staged activations are bf16 pairs laid out [k / 2][8 rows], one conflict-free 32-bit load per
// B fragment register.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void gemv_ldsm_x4_t(uint32_t addr, uint32_t (&a)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
}
__device__ __forceinline__ void gemv_mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MBLK>   // blocks of 8 activation rows: 1, 2 or 4 (M <= 8 * MBLK)
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_mma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ GemvParams p) {
  constexpr int COLS = 256;
  constexpr int XR = 8 * MBLK;   // 32-bit words per k pair in the staged activations
  extern __shared__ __align__(1024) uint8_t smem_mma[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_mma) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(tiles + GEMV_STAGES * GEMV_TILE_BYTES);  // [k/2][XR][2]
  __shared__ uint64_t full[GEMV_STAGES], empty[GEMV_STAGES];
  __shared__ float s_inv[32];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = p.M, N = p.N, K = p.K;
  const int col0 = blockIdx.x * COLS;
  const int k0 = blockIdx.y * p.k_per_split;            // a multiple of 32
  const int k1 = min(K, k0 + p.k_per_split);
  const int ntiles = (k1 - k0 + GEMV_KT - 1) / GEMV_KT;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_w);
    for (int s = 0; s < GEMV_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 8); }
    fence_barrier_init();
  }
  __syncthreads();

  float acc[2][MBLK][4];
#pragma unroll
  for (int nb = 0; nb < 2; ++nb)
#pragma unroll
    for (int mb = 0; mb < MBLK; ++mb)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[nb][mb][j] = 0.f;
  const int g = lane >> 2, tq = lane & 3;   // mma fragment coordinates of this lane

  if (warp == 8) {
    // ------------------------------ producer ------------------------------
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % GEMV_STAGES;
      if (t >= GEMV_STAGES && !mbar_wait(&empty[s], ((t / GEMV_STAGES) - 1) & 1, p.status, ST_TIMEOUT_EMPTY)) break;
      if (lane == 0) {
        // rows past K and columns past N arrive as zeros and still count towards the byte total
        mbar_arrive_expect_tx(&full[s], GEMV_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tma_load_2d(tiles + s * GEMV_TILE_BYTES + c * (GEMV_KT * 128), &tmap_w, &full[s], col0 + c * 64,
                      k0 + t * GEMV_KT);
      }
      __syncwarp();
    }
    pdl_wait();
  } else {
    // ------------------------------ consumers -----------------------------
    pdl_wait();   // X, the residual and the workspace belong to the previous kernel until here
    if (p.prologue == PRO_RMSNORM) {
      // row statistic with the association of rmsnorm_fwd_kernel (see the FMA kernel)
      float* s_part = reinterpret_cast<float*>(xs);   // [M][8 warps][32 lanes], overwritten by the staging below
      if (M == 1) {
        const __nv_bfloat16* xr = p.X;
        float a = 0.f;
        for (int c = lane * 8 + warp * 256; c < K; c += 8 * 256) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
          const float f[8] = {dbflo(raw.x), dbfhi(raw.x), dbflo(raw.y), dbfhi(raw.y),
                              dbflo(raw.z), dbfhi(raw.z), dbflo(raw.w), dbfhi(raw.w)};
#pragma unroll
          for (int j = 0; j < 8; ++j) a += f[j] * f[j];
        }
        s_part[warp * 32 + lane] = a;
      } else {
        // all rows of one column step are loaded before the first use; per row the adds keep their order
        float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int c = lane * 8 + warp * 256; c < K; c += 8 * 256) {
          uint4 raw[8];
#pragma unroll
          for (int m = 0; m < 8; ++m)
            if (m < M) raw[m] = *reinterpret_cast<const uint4*>(p.X + static_cast<size_t>(m) * p.ldx + c);
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            if (m < M) {
              const float f[8] = {dbflo(raw[m].x), dbfhi(raw[m].x), dbflo(raw[m].y), dbfhi(raw[m].y),
                                  dbflo(raw[m].z), dbfhi(raw[m].z), dbflo(raw[m].w), dbfhi(raw[m].w)};
#pragma unroll
              for (int j = 0; j < 8; ++j) a8[m] += f[j] * f[j];
            }
          }
        }
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < M) s_part[(m * 8 + warp) * 32 + lane] = a8[m];
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (warp < M) {
        float ss = s_part[(warp * 8) * 32 + lane];
#pragma unroll
        for (int a = 1; a < 8; ++a) ss += s_part[(warp * 8 + a) * 32 + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_inv[warp] = rsqrtf(ss / static_cast<float>(K) + p.eps);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    // stage f(X) as bf16 pairs: (k, k + 1) of row m in the 32-bit word (k / 2) * 8 + m. Only the M live rows are
    // written (lanes of the other rows feed zeros to the MMA below); k past the split's range is zero, since a
    // weight row past K is zero too and 0 * x must not meet garbage
    uint32_t* xs_w = reinterpret_cast<uint32_t*>(xs);
    const int n_pairs = ntiles * GEMV_KT / 2;
    const bool vec_ok = ((p.ldx & 7) == 0) && ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.X) & 15) == 0) &&
                        (p.prologue != PRO_RMSNORM || (reinterpret_cast<uintptr_t>(p.norm_w) & 15) == 0);
    if (vec_ok && M > 1) {   // a single row is staged faster by the pair loop below (3.40 against 4.07 ms per decode step)
      // eight consecutive k of one row per thread: one 16-byte load of X (and of the gain, or of the up half)
      const int n_oct = n_pairs / 4;
      for (int i = threadIdx.x; i < n_oct * M; i += 256) {
        const int ko = i / M, m = i - ko * M;
        const int k = k0 + ko * 8;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
        if (k < k1) {      // k1 - k0 and K are multiples of 8: an octet is inside the range or outside it
          const __nv_bfloat16* xr = p.X + static_cast<size_t>(m) * p.ldx + k;
          const uint4 raw = *reinterpret_cast<const uint4*>(xr);
          v[0] = dbflo(raw.x); v[1] = dbfhi(raw.x); v[2] = dbflo(raw.y); v[3] = dbfhi(raw.y);
          v[4] = dbflo(raw.z); v[5] = dbfhi(raw.z); v[6] = dbflo(raw.w); v[7] = dbfhi(raw.w);
          if (p.prologue == PRO_RMSNORM) {
            const uint4 gw = *reinterpret_cast<const uint4*>(p.norm_w + k);
            const float g[8] = {dbflo(gw.x), dbfhi(gw.x), dbflo(gw.y), dbfhi(gw.y),
                                dbflo(gw.z), dbfhi(gw.z), dbflo(gw.w), dbfhi(gw.w)};
            const float inv = s_inv[m];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * inv * g[e];
          } else if (p.prologue == PRO_SWIGLU) {
            const uint4 uw = *reinterpret_cast<const uint4*>(xr + K);
            const float u[8] = {dbflo(uw.x), dbfhi(uw.x), dbflo(uw.y), dbfhi(uw.y),
                                dbflo(uw.z), dbfhi(uw.z), dbflo(uw.w), dbfhi(uw.w)};
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] / (1.f + __expf(-v[e])) * u[e];
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) xs_w[(ko * 4 + e) * XR + m] = dpack(v[2 * e], v[2 * e + 1]);
      }
    } else {
      for (int i = threadIdx.x; i < n_pairs * M; i += 256) {
        const int kp = i / M, m = i - kp * M;
        float xv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int k = k0 + kp * 2 + e;
          float v = 0.f;
          if (k < k1) {
            v = __bfloat162float(p.X[static_cast<size_t>(m) * p.ldx + k]);
            if (p.prologue == PRO_RMSNORM) {
              v = v * s_inv[m] * __bfloat162float(p.norm_w[k]);
            } else if (p.prologue == PRO_SWIGLU) {
              const float u = __bfloat162float(p.X[static_cast<size_t>(m) * p.ldx + K + k]);
              v = v / (1.f + __expf(-v)) * u;
            }
          }
          xv[e] = v;
        }
        xs_w[kp * XR + m] = dpack(xv[0], xv[1]);
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    const uint32_t* xs32 = reinterpret_cast<const uint32_t*>(xs);
    // ldmatrix lane address: matrix mi = lane / 8 -> (k group = mi / 2, n half = mi % 2), row lane % 8
    const int mi = lane >> 3, lr = lane & 7;
    const int sub = warp >> 1;                          // which 64-column box holds this warp's columns
    const uint32_t tiles_u32 = smem_u32(tiles) + sub * (GEMV_KT * 128);
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % GEMV_STAGES;
      if (!mbar_wait(&full[s], (t / GEMV_STAGES) & 1, p.status, ST_TIMEOUT_FULL)) break;
      const uint32_t tbase = tiles_u32 + s * GEMV_TILE_BYTES;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const int kp = (t * GEMV_KT + ks * 16) >> 1;      // index of the first bf16 pair of this k-step
        uint32_t b0[MBLK], b1[MBLK];
#pragma unroll
        for (int mb = 0; mb < MBLK; ++mb) {
          const bool live = mb * 8 + g < M;
          b0[mb] = live ? xs32[(kp + tq) * XR + mb * 8 + g] : 0u;
          b1[mb] = live ? xs32[(kp + 4 + tq) * XR + mb * 8 + g] : 0u;
        }
        const int r = ks * 16 + (mi >> 1) * 8 + lr;       // k row inside the tile
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          const int chunk = (warp & 1) * 4 + nb * 2 + (mi & 1);   // 16-byte chunk of the 128-byte row
          uint32_t a[4];
          gemv_ldsm_x4_t(tbase + r * 128 + ((chunk ^ (r & 7)) << 4), a);
#pragma unroll
          for (int mb = 0; mb < MBLK; ++mb) gemv_mma_16816(acc[nb][mb], a, b0[mb], b1[mb]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  __syncthreads();
  pdl_trigger();
  const bool direct = gridDim.y == 1;
  const bool coll = p.coll.W > 1;
  const bool amax = p.amax.out_tokens != nullptr;
  float* vals = reinterpret_cast<float*>(tiles);   // [M][COLS]: the ring is idle from here on
  // the epoch word is advanced only after every finishing CTA of this call has read it
  const uint32_t epoch = coll ? *reinterpret_cast<volatile uint32_t*>(p.coll.epoch_word) + 1u : 0u;
  if (warp < 8) {
    // accumulator (nb, mb, j): column col0 + 32 warp + 16 nb + g + 8 (j / 2), row 8 mb + 2 tq + (j & 1)
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int mb = 0; mb < MBLK; ++mb) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int gc = col0 + warp * 32 + nb * 16 + g + (j >> 1) * 8;
          const int m = mb * 8 + tq * 2 + (j & 1);
          if (m < M && gc < N) {
            float sum = acc[nb][mb][j];
            if (direct) {
              if (coll) { gemv_coll_push(p, epoch, m, gc, sum); continue; }
              if (p.R) sum += __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]);
              if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(sum);
              if (p.out_f32) p.out_f32[static_cast<size_t>(m) * N + gc] = sum;
              if (amax) vals[m * COLS + (gc - col0)] = sum;
            } else {
              p.part[(static_cast<size_t>(blockIdx.y) * M + m) * N + gc] = sum;
            }
          }
        }
      }
    }
  }
  if (direct) {
    if (coll) gemv_coll_finish(p, epoch, col0, min(COLS, N - col0), &s_last);
    else if (amax) gemv_argmax_tail(p, vals, COLS, col0, min(COLS, N - col0), &s_last);
    return;
  }
  // split-K finish by the last CTA of this column block
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.counters + blockIdx.x, 1u);
    s_last = (prev == gridDim.y - 1) ? 1 : 0;
    if (s_last) p.counters[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int ncols = min(COLS, N - col0);
  for (int i = threadIdx.x; i < M * ncols; i += GEMV_THREADS) {
    const int m = i / ncols, gc = col0 + (i - m * ncols);
    float sum = 0.f;
    const float* pp = p.part + static_cast<size_t>(m) * N + gc;
    const size_t pstride = static_cast<size_t>(M) * N;
    const int ns = static_cast<int>(gridDim.y);
    for (int k = 0; k < ns; k += 8) {   // eight loads in flight, added in split order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (k + u < ns) ? __ldcg(pp + (k + u) * pstride) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) if (k + u < ns) sum += v[u];
    }
    if (coll) { gemv_coll_push(p, epoch, m, gc, sum); continue; }
    if (p.R) sum += __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]);
    if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(sum);
    if (p.out_f32) p.out_f32[static_cast<size_t>(m) * N + gc] = sum;
    if (amax) vals[m * COLS + (gc - col0)] = sum;
  }
  if (coll) gemv_coll_finish(p, epoch, col0, ncols, &s_last);
  else if (amax) gemv_argmax_tail(p, vals, COLS, col0, ncols, &s_last);
}

// fp16 pair of two values that are first rounded to bf16 (the activation format) and saturated to the fp16 range
__device__ __forceinline__ uint32_t hpack_bf16_rounded(float a, float b) {
  const float c0 = fminf(fmaxf(__bfloat162float(__float2bfloat16_rn(a)), -65504.f), 65504.f);
  const float c1 = fminf(fmaxf(__bfloat162float(__float2bfloat16_rn(b)), -65504.f), 65504.f);
  const __half2 hp = __floats2half2_rn(c0, c1);
  return *reinterpret_cast<const uint32_t*>(&hp);
}

// int8 weights on the same tensor-core path: the tile is streamed as 16-bit words (two int8 columns per word) in
// 128-byte-swizzled boxes, the transposed ldmatrix hands every thread 2 x 2 (k, column) bytes, a byte permute and one
// packed fp16 subtract turn them into exact fp16 values, and the MMA runs in fp16 with fp32 accumulation; the
// activations are the bf16-rounded values carried as fp16. The column scales are applied after the sum.
__device__ __forceinline__ void gemv_mma_16816_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(GEMV_THREADS)
gemv_mma_i8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ GemvParams p) {
  constexpr int COLS = 512;      // int8 columns per CTA: 512 bytes of every weight row
  constexpr int MBLK = 1;
  constexpr int XR = 8;          // 32-bit words (fp16 pairs) per k pair in the staged activations
  extern __shared__ __align__(1024) uint8_t smem_mma[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_mma) + 1023) & ~uintptr_t(1023));
  __half* xs = reinterpret_cast<__half*>(tiles + GEMV_STAGES * GEMV_TILE_BYTES);  // [k/2][XR][2] fp16
  __shared__ uint64_t full[GEMV_STAGES], empty[GEMV_STAGES];
  __shared__ float s_inv[32];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = p.M, N = p.N, K = p.K;
  const int col0 = blockIdx.x * COLS;
  const int k0 = blockIdx.y * p.k_per_split;            // a multiple of 32
  const int k1 = min(K, k0 + p.k_per_split);
  const int ntiles = (k1 - k0 + GEMV_KT - 1) / GEMV_KT;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_w);
    for (int s = 0; s < GEMV_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 8); }
    fence_barrier_init();
  }
  __syncthreads();

  float acc[4][MBLK][4];
#pragma unroll
  for (int nb = 0; nb < 4; ++nb)
#pragma unroll
    for (int mb = 0; mb < MBLK; ++mb)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[nb][mb][j] = 0.f;
  const int g = lane >> 2, tq = lane & 3;   // mma fragment coordinates of this lane

  if (warp == 8) {
    // ------------------------------ producer ------------------------------
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % GEMV_STAGES;
      if (t >= GEMV_STAGES && !mbar_wait(&empty[s], ((t / GEMV_STAGES) - 1) & 1, p.status, ST_TIMEOUT_EMPTY)) break;
      if (lane == 0) {
        // rows past K and columns past N arrive as zeros and still count towards the byte total
        mbar_arrive_expect_tx(&full[s], GEMV_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tma_load_2d(tiles + s * GEMV_TILE_BYTES + c * (GEMV_KT * 128), &tmap_w, &full[s], col0 / 2 + c * 64,
                      k0 + t * GEMV_KT);   // the map is over 16-bit words: 64 words = 128 int8 columns
      }
      __syncwarp();
    }
    pdl_wait();
  } else {
    // ------------------------------ consumers -----------------------------
    pdl_wait();   // X, the residual and the workspace belong to the previous kernel until here
    if (p.prologue == PRO_RMSNORM) {
      // row statistic with the association of rmsnorm_fwd_kernel (see the FMA kernel)
      float* s_part = reinterpret_cast<float*>(xs);   // [M][8 warps][32 lanes], overwritten by the staging below
      if (M == 1) {
        const __nv_bfloat16* xr = p.X;
        float a = 0.f;
        for (int c = lane * 8 + warp * 256; c < K; c += 8 * 256) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
          const float f[8] = {dbflo(raw.x), dbfhi(raw.x), dbflo(raw.y), dbfhi(raw.y),
                              dbflo(raw.z), dbfhi(raw.z), dbflo(raw.w), dbfhi(raw.w)};
#pragma unroll
          for (int j = 0; j < 8; ++j) a += f[j] * f[j];
        }
        s_part[warp * 32 + lane] = a;
      } else {
        // all rows of one column step are loaded before the first use; per row the adds keep their order
        float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int c = lane * 8 + warp * 256; c < K; c += 8 * 256) {
          uint4 raw[8];
#pragma unroll
          for (int m = 0; m < 8; ++m)
            if (m < M) raw[m] = *reinterpret_cast<const uint4*>(p.X + static_cast<size_t>(m) * p.ldx + c);
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            if (m < M) {
              const float f[8] = {dbflo(raw[m].x), dbfhi(raw[m].x), dbflo(raw[m].y), dbfhi(raw[m].y),
                                  dbflo(raw[m].z), dbfhi(raw[m].z), dbflo(raw[m].w), dbfhi(raw[m].w)};
#pragma unroll
              for (int j = 0; j < 8; ++j) a8[m] += f[j] * f[j];
            }
          }
        }
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < M) s_part[(m * 8 + warp) * 32 + lane] = a8[m];
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (warp < M) {
        float ss = s_part[(warp * 8) * 32 + lane];
#pragma unroll
        for (int a = 1; a < 8; ++a) ss += s_part[(warp * 8 + a) * 32 + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_inv[warp] = rsqrtf(ss / static_cast<float>(K) + p.eps);
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    // stage f(X) as fp16 pairs (of the bf16-rounded value, saturated to the fp16 range): (k, k + 1) of row m in the
    // 32-bit word (k / 2) * 8 + m. Only the M live rows are
    // written (lanes of the other rows feed zeros to the MMA below); k past the split's range is zero, since a
    // weight row past K is zero too and 0 * x must not meet garbage
    uint32_t* xs_w = reinterpret_cast<uint32_t*>(xs);
    const int n_pairs = ntiles * GEMV_KT / 2;
    const bool vec_ok = ((p.ldx & 7) == 0) && ((K & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.X) & 15) == 0) &&
                        (p.prologue != PRO_RMSNORM || (reinterpret_cast<uintptr_t>(p.norm_w) & 15) == 0);
    if (vec_ok && M > 1) {   // a single row is staged faster by the pair loop below (3.40 against 4.07 ms per decode step)
      // eight consecutive k of one row per thread: one 16-byte load of X (and of the gain, or of the up half)
      const int n_oct = n_pairs / 4;
      for (int i = threadIdx.x; i < n_oct * M; i += 256) {
        const int ko = i / M, m = i - ko * M;
        const int k = k0 + ko * 8;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
        if (k < k1) {      // k1 - k0 and K are multiples of 8: an octet is inside the range or outside it
          const __nv_bfloat16* xr = p.X + static_cast<size_t>(m) * p.ldx + k;
          const uint4 raw = *reinterpret_cast<const uint4*>(xr);
          v[0] = dbflo(raw.x); v[1] = dbfhi(raw.x); v[2] = dbflo(raw.y); v[3] = dbfhi(raw.y);
          v[4] = dbflo(raw.z); v[5] = dbfhi(raw.z); v[6] = dbflo(raw.w); v[7] = dbfhi(raw.w);
          if (p.prologue == PRO_RMSNORM) {
            const uint4 gw = *reinterpret_cast<const uint4*>(p.norm_w + k);
            const float g[8] = {dbflo(gw.x), dbfhi(gw.x), dbflo(gw.y), dbfhi(gw.y),
                                dbflo(gw.z), dbfhi(gw.z), dbflo(gw.w), dbfhi(gw.w)};
            const float inv = s_inv[m];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * inv * g[e];
          } else if (p.prologue == PRO_SWIGLU) {
            const uint4 uw = *reinterpret_cast<const uint4*>(xr + K);
            const float u[8] = {dbflo(uw.x), dbfhi(uw.x), dbflo(uw.y), dbfhi(uw.y),
                                dbflo(uw.z), dbfhi(uw.z), dbflo(uw.w), dbfhi(uw.w)};
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] / (1.f + __expf(-v[e])) * u[e];
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) xs_w[(ko * 4 + e) * XR + m] = hpack_bf16_rounded(v[2 * e], v[2 * e + 1]);
      }
    } else {
      for (int i = threadIdx.x; i < n_pairs * M; i += 256) {
        const int kp = i / M, m = i - kp * M;
        float xv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int k = k0 + kp * 2 + e;
          float v = 0.f;
          if (k < k1) {
            v = __bfloat162float(p.X[static_cast<size_t>(m) * p.ldx + k]);
            if (p.prologue == PRO_RMSNORM) {
              v = v * s_inv[m] * __bfloat162float(p.norm_w[k]);
            } else if (p.prologue == PRO_SWIGLU) {
              const float u = __bfloat162float(p.X[static_cast<size_t>(m) * p.ldx + K + k]);
              v = v / (1.f + __expf(-v)) * u;
            }
          }
          xv[e] = v;
        }
        xs_w[kp * XR + m] = hpack_bf16_rounded(xv[0], xv[1]);
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    const uint32_t* xs32 = reinterpret_cast<const uint32_t*>(xs);
    // ldmatrix lane address: matrix mi = lane / 8 -> (n block of the pair = mi / 2, k group = mi % 2), row lane % 8.
    // A 16-bit unit holds two int8 columns, so one transposed 8x8 matrix spans 16 columns x 8 k: the thread gets
    // bytes {W[2tq][2g], W[2tq][2g+1], W[2tq+1][2g], W[2tq+1][2g+1]}; the even column feeds MMA row g, the odd one
    // row g + 8 (the epilogue maps rows back to columns).
    const int mi = lane >> 3, lr = lane & 7;
    const int sub = warp >> 1;                          // which 128-column box holds this warp's 64 columns
    const uint32_t tiles_u32 = smem_u32(tiles) + sub * (GEMV_KT * 128);
    const __half2 bias = __floats2half2_rn(1152.f, 1152.f);   // 1024 (the magic exponent) + 128 (the sign flip)
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % GEMV_STAGES;
      if (!mbar_wait(&full[s], (t / GEMV_STAGES) & 1, p.status, ST_TIMEOUT_FULL)) break;
      const uint32_t tbase = tiles_u32 + s * GEMV_TILE_BYTES;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const int kp = (t * GEMV_KT + ks * 16) >> 1;      // index of the first fp16 pair of this k-step
        const bool live = g < M;
        const uint32_t b0 = live ? xs32[(kp + tq) * XR + g] : 0u;
        const uint32_t b1 = live ? xs32[(kp + 4 + tq) * XR + g] : 0u;
        const int r = ks * 16 + (mi & 1) * 8 + lr;        // k row inside the tile
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {                  // two n blocks of 16 columns per ldmatrix.x4
          const int chunk = (warp & 1) * 4 + pr * 2 + (mi >> 1);   // 16-byte chunk = 16 int8 columns
          uint32_t raw[4];
          gemv_ldsm_x4_t(tbase + r * 128 + ((chunk ^ (r & 7)) << 4), raw);
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2) {
            // int8 -> fp16 without the conversion pipe: flip the sign bit (value + 128 as an unsigned byte), drop the
            // byte into the mantissa of 1024.0 and subtract 1152
            const uint32_t u_lo = raw[q2 * 2] ^ 0x80808080u, u_hi = raw[q2 * 2 + 1] ^ 0x80808080u;
            uint32_t a[4];
            a[0] = __byte_perm(u_lo, 0x64646464u, 0x4240);   // row g     (even column), k 0-7
            a[1] = __byte_perm(u_lo, 0x64646464u, 0x4341);   // row g + 8 (odd column),  k 0-7
            a[2] = __byte_perm(u_hi, 0x64646464u, 0x4240);   // k 8-15
            a[3] = __byte_perm(u_hi, 0x64646464u, 0x4341);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __half2 h = *reinterpret_cast<__half2*>(&a[e]);
              h = __hsub2(h, bias);
              a[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            gemv_mma_16816_f16(acc[pr * 2 + q2][0], a, b0, b1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  __syncthreads();
  pdl_trigger();
  const bool direct = gridDim.y == 1;
  const bool coll = p.coll.W > 1;
  const bool amax = p.amax.out_tokens != nullptr;
  float* vals = reinterpret_cast<float*>(tiles);   // [M][COLS]: the ring is idle from here on
  // the epoch word is advanced only after every finishing CTA of this call has read it
  const uint32_t epoch = coll ? *reinterpret_cast<volatile uint32_t*>(p.coll.epoch_word) + 1u : 0u;
  if (warp < 8) {
    // accumulator (nb, j): column col0 + 64 warp + 16 nb + 2 g + (j / 2), row 2 tq + (j & 1)
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gc = col0 + warp * 64 + nb * 16 + 2 * g + (j >> 1);
        const int m = tq * 2 + (j & 1);
        if (m < M && gc < N) {
          float sum = acc[nb][0][j];
          if (direct) {
            sum *= p.scale[gc];
            if (coll) { gemv_coll_push(p, epoch, m, gc, sum); continue; }
            if (p.R) sum += __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]);
            if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(sum);
            if (p.out_f32) p.out_f32[static_cast<size_t>(m) * N + gc] = sum;
            if (amax) vals[m * COLS + (gc - col0)] = sum;
          } else {
            p.part[(static_cast<size_t>(blockIdx.y) * M + m) * N + gc] = sum;
          }
        }
      }
    }
  }
  if (direct) {
    if (coll) gemv_coll_finish(p, epoch, col0, min(COLS, N - col0), &s_last);
    else if (amax) gemv_argmax_tail(p, vals, COLS, col0, min(COLS, N - col0), &s_last);
    return;
  }
  // split-K finish by the last CTA of this column block
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.counters + blockIdx.x, 1u);
    s_last = (prev == gridDim.y - 1) ? 1 : 0;
    if (s_last) p.counters[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int ncols = min(COLS, N - col0);
  for (int i = threadIdx.x; i < M * ncols; i += GEMV_THREADS) {
    const int m = i / ncols, gc = col0 + (i - m * ncols);
    float sum = 0.f;
    const float* pp = p.part + static_cast<size_t>(m) * N + gc;
    const size_t pstride = static_cast<size_t>(M) * N;
    const int ns = static_cast<int>(gridDim.y);
    for (int k = 0; k < ns; k += 8) {   // eight loads in flight, added in split order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (k + u < ns) ? __ldcg(pp + (k + u) * pstride) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) if (k + u < ns) sum += v[u];
    }
    sum *= p.scale[gc];
    if (coll) { gemv_coll_push(p, epoch, m, gc, sum); continue; }
    if (p.R) sum += __bfloat162float(p.R[static_cast<size_t>(m) * p.ldr + gc]);
    if (p.out) p.out[static_cast<size_t>(m) * p.ldo + gc] = __float2bfloat16_rn(sum);
    if (p.out_f32) p.out_f32[static_cast<size_t>(m) * N + gc] = sum;
    if (amax) vals[m * COLS + (gc - col0)] = sum;
  }
  if (coll) gemv_coll_finish(p, epoch, col0, ncols, &s_last);
  else if (amax) gemv_argmax_tail(p, vals, COLS, col0, ncols, &s_last);
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
  // grid = (n_tok, H + 2*Hkv): one CTA per head of one token, one thread per (even, odd) pair
  const int t = blockIdx.x, head = blockIdx.y;
  if (t >= n_tok) return;
  pdl_wait();
  const int b = seq_of[t], p = pos[t];
  const int half = dh >> 1;
  const int pr = threadIdx.x;
  if (pr >= half) return;
  uint32_t* e = reinterpret_cast<uint32_t*>(qkv + static_cast<size_t>(t) * ld + head * dh) + pr;
  uint32_t v = *e;
  if (head < H + Hkv) {   // query and key heads rotate
    const float c = cos_t[static_cast<size_t>(p) * half + pr], s = sin_t[static_cast<size_t>(p) * half + pr];
    const float x0 = dbflo(v), x1 = dbfhi(v);
    v = dpack(x0 * c - x1 * s, x0 * s + x1 * c);
    *e = v;
  }
  if (head >= H) {        // key and value heads go to the cache
    const int kv = head >= H + Hkv ? 1 : 0;
    const int h = head - H - kv * Hkv;
    const int blk = block_table[b * max_blocks + p / page];
    const int slot = p % page;
    uint32_t* dst = reinterpret_cast<uint32_t*>(
        pool + ((((static_cast<size_t>(blk) * 2 + kv) * Hkv + h) * page + slot) * dh)) + pr;
    *dst = v;
  }
}

// ---------------------------------------------------------------------------
// Split-KV GQA flash-decode. grid = (Hkv, B, n_splits); 128 threads = 4 warps.
// A CTA serves the G = H/Hkv (<= 16) query heads of one kv head for one sequence over the kv
// positions of its split. K/V rows stream through a two-stage ring of 64-position tiles
// (cp.async, 16-byte padded rows so ldmatrix is conflict-free); warp w owns positions
// [16w, 16w+16) of every tile and runs them as m16n8k16 tensor-core products: the G query heads are
// the 16 rows of the A operand (unused rows zero), S = Q K^T in two 16x8 blocks, online softmax on
// the accumulator fragments, P re-used in registers as the A operand of O += P V.
// At the end the four warps' (m, l, O) are merged in warp order through shared memory; the split
// partials are merged in split order by the LAST CTA of each (sequence, kv head) (a counter, no
// data atomics), so there is one launch and the summation tree depends only on (L, n_splits).
// ---------------------------------------------------------------------------
constexpr int DEC_TK = 64;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t n = valid ? 16u : 0u;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct DecodeAttnParams {
  const __nv_bfloat16* q; int ldq;
  const __nv_bfloat16* pool;
  const int* block_table; int max_blocks, page;
  const int* seq_len;
  int H, Hkv, n_splits;
  float scale_log2;
  float* part_o;    // [B, H, n_splits, dh]
  float* part_ml;   // [B, H, n_splits, 2]
  __nv_bfloat16* out; int ldo;
  unsigned int* counters;  // [B * Hkv], zero between calls
};

template <int DH>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __grid_constant__ DecodeAttnParams p) {
  constexpr int ROWB = DH * 2 + 16;            // padded row pitch in bytes
  constexpr int TILE_B = DEC_TK * ROWB;        // one K (or V) tile
  constexpr int KS = DH / 16;                  // k-steps of Q K^T
  constexpr int NB = DH / 8;                   // 8-wide output blocks of P V
  constexpr int CH = DH / 8;                   // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t smem[];   // [2 stages][K tile | V tile]
  __shared__ int s_last;
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int H = p.H, Hkv = p.Hkv, G = H / Hkv, n_splits = p.n_splits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, tq = lane & 3;
  pdl_wait();
  const int L = p.seq_len[b];
  const int per_split = ((L + n_splits - 1) / n_splits + DEC_TK - 1) / DEC_TK * DEC_TK;
  const int p0 = split * per_split;
  const int p1 = min(L, p0 + per_split);
  const int ntiles = p1 > p0 ? (p1 - p0 + DEC_TK - 1) / DEC_TK : 0;
  const size_t vofs = static_cast<size_t>(Hkv) * p.page * DH;

  auto load_tile = [&](int t, int stage) {
    uint8_t* kt = smem + stage * 2 * TILE_B;
    uint8_t* vt = kt + TILE_B;
    const int t0 = p0 + t * DEC_TK;
    for (int i = threadIdx.x; i < DEC_TK * CH; i += 128) {
      const int r = i / CH, c = i - r * CH;
      const int pos = t0 + r;
      const bool valid = pos < p1;
      const int pp = valid ? pos : p0;
      const int blk = p.block_table[b * p.max_blocks + pp / p.page];
      const __nv_bfloat16* src =
          p.pool + (((static_cast<size_t>(blk) * 2) * Hkv + kvh) * p.page + pp % p.page) * DH + c * 8;
      cp_async16(kt + r * ROWB + c * 16, src, valid);
      cp_async16(vt + r * ROWB + c * 16, src + vofs, valid);
    }
  };

  if (ntiles > 0) load_tile(0, 0);
  cp_async_commit();

  // Q as A fragments: row `quad` (and quad + 8) of the 16-row operand is query head kvh*G + row
  uint32_t qa[KS][4];
  {
    const __nv_bfloat16* q_lo = p.q + static_cast<size_t>(b) * p.ldq + static_cast<size_t>(kvh * G + quad) * DH;
    const __nv_bfloat16* q_hi = q_lo + 8 * DH;
    const bool lo = quad < G, hi = quad + 8 < G;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + tq * 2;
      qa[ks][0] = lo ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
      qa[ks][1] = hi ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
      qa[ks][2] = lo ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
      qa[ks][3] = hi ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
    }
  }
  float m_lo = -1.0e30f, m_hi = -1.0e30f, l_lo = 0.f, l_hi = 0.f;
  float o[NB][4];
#pragma unroll
  for (int j = 0; j < NB; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

  for (int t = 0; t < ntiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < ntiles) load_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kt = smem_u32(smem + stage * 2 * TILE_B);
    const uint32_t vt = kt + TILE_B;
    const int t0 = p0 + t * DEC_TK;
    // ---- S = Q K^T for this warp's 16 positions (two 16x8 blocks) ----
    float sacc[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) { sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f; }
    {
      const int mi = lane >> 3;  // matrix index of the x4 load: block = mi / 2, k half = mi % 2
      const uint32_t base = kt + (warp * 16 + (mi >> 1) * 8 + (lane & 7)) * ROWB + (mi & 1) * 16;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t r0, r1, r2, r3;
        ldsm_x4(base + ks * 32, r0, r1, r2, r3);
        mma_16816(sacc[0], qa[ks], r0, r1);
        mma_16816(sacc[1], qa[ks], r2, r3);
      }
    }
    // ---- online softmax on the fragments ----
    float mx_lo = -1.0e30f, mx_hi = -1.0e30f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int pos = t0 + warp * 16 + nb * 8 + tq * 2;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool ok = pos + e < p1;
        sacc[nb][e] = ok ? sacc[nb][e] * p.scale_log2 : -1.0e30f;
        sacc[nb][2 + e] = ok ? sacc[nb][2 + e] * p.scale_log2 : -1.0e30f;
        mx_lo = fmaxf(mx_lo, sacc[nb][e]);
        mx_hi = fmaxf(mx_hi, sacc[nb][2 + e]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float al_lo = exp2f(m_lo - mn_lo), al_hi = exp2f(m_hi - mn_hi);
    m_lo = mn_lo; m_hi = mn_hi;
    uint32_t pa[4];
    {
      float pr[2][4];
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          // a masked score stays at -1e30: exp2 of (-1e30 - m) is 0 unless the row is empty so far,
          // in which case m is -1e30 too and the position must still contribute nothing
          pr[nb][e] = sacc[nb][e] > -1.0e29f ? exp2f(sacc[nb][e] - mn_lo) : 0.f;
          pr[nb][2 + e] = sacc[nb][2 + e] > -1.0e29f ? exp2f(sacc[nb][2 + e] - mn_hi) : 0.f;
          sum_lo += pr[nb][e];
          sum_hi += pr[nb][2 + e];
        }
      }
      l_lo = l_lo * al_lo + sum_lo;
      l_hi = l_hi * al_hi + sum_hi;
      pa[0] = dpack(pr[0][0], pr[0][1]);
      pa[1] = dpack(pr[0][2], pr[0][3]);
      pa[2] = dpack(pr[1][0], pr[1][1]);
      pa[3] = dpack(pr[1][2], pr[1][3]);
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) { o[j][0] *= al_lo; o[j][1] *= al_lo; o[j][2] *= al_hi; o[j][3] *= al_hi; }
    // ---- O += P V over this warp's 16 positions ----
    {
      const int mi = lane >> 3;  // k half = mi % 2, output block offset = mi / 2
      const uint32_t base = vt + (warp * 16 + (mi & 1) * 8 + (lane & 7)) * ROWB + (mi >> 1) * 16;
#pragma unroll
      for (int j = 0; j < NB; j += 2) {
        uint32_t r0, r1, r2, r3;
        ldsm_x4_t(base + j * 16, r0, r1, r2, r3);
        mma_16816(o[j], pa, r0, r1);
        mma_16816(o[j + 1], pa, r2, r3);
      }
    }
    __syncthreads();   // the stage is refilled by the next iteration's load
  }
  cp_async_wait<0>();
  __syncthreads();
  pdl_trigger();   // the output projection may start prefetching its weights

  // ---- merge the four warps in warp order ----
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float* sm_o = reinterpret_cast<float*>(smem);           // [4 warps][16 rows][DH]
  float* sm_ml = sm_o + 4 * 16 * DH;                      // [4 warps][16 rows][2]
#pragma unroll
  for (int j = 0; j < NB; ++j) {
    float* r_lo = sm_o + (warp * 16 + quad) * DH + j * 8 + tq * 2;
    float* r_hi = r_lo + 8 * DH;
    r_lo[0] = o[j][0]; r_lo[1] = o[j][1];
    r_hi[0] = o[j][2]; r_hi[1] = o[j][3];
  }
  if (tq == 0) {
    sm_ml[(warp * 16 + quad) * 2] = m_lo;      sm_ml[(warp * 16 + quad) * 2 + 1] = l_lo;
    sm_ml[(warp * 16 + quad + 8) * 2] = m_hi;  sm_ml[(warp * 16 + quad + 8) * 2 + 1] = l_hi;
  }
  __syncthreads();
  const bool direct = n_splits == 1;
  for (int i = threadIdx.x; i < G * DH; i += 128) {
    const int g = i / DH, d = i - g * DH;
    float mt = -1.0e30f;
#pragma unroll
    for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sm_ml[(w * 16 + g) * 2]);
    float lt = 0.f, ot = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f(sm_ml[(w * 16 + g) * 2] - mt);
      lt += sm_ml[(w * 16 + g) * 2 + 1] * wgt;
      ot += sm_o[(w * 16 + g) * DH + d] * wgt;
    }
    const int h = kvh * G + g;
    if (direct) {
      p.out[static_cast<size_t>(b) * p.ldo + h * DH + d] = __float2bfloat16_rn(lt > 0.f ? ot / lt : 0.f);
    } else {
      const size_t idx = (static_cast<size_t>(b) * H + h) * n_splits + split;
      p.part_o[idx * DH + d] = ot;
      if (d == 0) { p.part_ml[idx * 2] = mt; p.part_ml[idx * 2 + 1] = lt; }
    }
  }
  if (direct) return;
  // ---- the last CTA of this (sequence, kv head) merges the splits in split order ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* ctr = p.counters + b * Hkv + kvh;
    const unsigned int prev = atomicAdd(ctr, 1u);
    s_last = (prev == static_cast<unsigned int>(n_splits) - 1) ? 1 : 0;
    if (s_last) *ctr = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < G * DH; i += 128) {
    const int g = i / DH, d = i - g * DH;
    const int h = kvh * G + g;
    const size_t bh = static_cast<size_t>(b) * H + h;
    const float* ml = p.part_ml + bh * n_splits * 2;
    const float* po = p.part_o + bh * n_splits * DH + d;
    float mt = -1.0e30f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (s0 + u < n_splits) ? __ldcg(ml + (s0 + u) * 2) : -1.0e30f;
#pragma unroll
      for (int u = 0; u < 8; ++u) mt = fmaxf(mt, v[u]);
    }
    float lt = 0.f, ot = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {   // eight splits' loads in flight, added in split order
      float vm[8], vl[8], vo[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool ok = s0 + u < n_splits;
        vm[u] = ok ? __ldcg(ml + (s0 + u) * 2) : -1.0e30f;
        vl[u] = ok ? __ldcg(ml + (s0 + u) * 2 + 1) : 0.f;
        vo[u] = ok ? __ldcg(po + static_cast<size_t>(s0 + u) * DH) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < n_splits) {
          const float wgt = exp2f(vm[u] - mt);
          lt += vl[u] * wgt;
          ot += vo[u] * wgt;
        }
      }
    }
    p.out[static_cast<size_t>(b) * p.ldo + h * DH + d] = __float2bfloat16_rn(lt > 0.f ? ot / lt : 0.f);
  }
}

// ---------------------------------------------------------------------------
// Arg-max over logits rows with the rule of the reference's greedy loop (`best = row[0]; if v > best`,
// scirust-cuda/src/decode.rs:107-114): a NaN in column 0 makes token 0 win outright; any other NaN is
// skipped explicitly (`v != v`), never left to how a comparison with NaN folds; among equal maxima the
// lowest index wins. Two stages.
// Stage 1: each CTA scans a slab of `cols_per_cta` columns of one row -> (value, index), index
// 0x7fffffff when the slab holds no number.
// Stage 2: one thread per row picks the best slab result and writes the token to `out_tokens[row]`
// (int64, the device-side feedback buffer) and optionally appends it to `generated[row, step]`.
// ---------------------------------------------------------------------------
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int V, int cols_per_cta,
                                      float* __restrict__ pval, int* __restrict__ pidx) {
  __shared__ float sv[256];
  __shared__ int si[256];
  const int row = blockIdx.y, slab = blockIdx.x;
  const int c0 = slab * cols_per_cta, c1 = min(V, c0 + cols_per_cta);
  const float* lr = logits + static_cast<size_t>(row) * V;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = c0 + threadIdx.x; c < c1; c += 256) {
    const float v = lr[c];
    if (v != v) continue;
    if (argmax_better(v, c, best, bi)) { best = v; bi = c; }
  }
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float bb = sv[threadIdx.x + s];
      const int ib = si[threadIdx.x + s];
      if (argmax_better(bb, ib, sv[threadIdx.x], si[threadIdx.x])) { sv[threadIdx.x] = bb; si[threadIdx.x] = ib; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    pval[row * gridDim.x + slab] = sv[0];
    pidx[row * gridDim.x + slab] = si[0];
  }
}
__global__ void argmax_final_kernel(const float* __restrict__ logits, int V, const float* __restrict__ pval,
                                    const int* __restrict__ pidx, int n_slabs, int64_t* __restrict__ out_tokens,
                                    int64_t* __restrict__ generated, int gen_stride, int step) {
  const int row = blockIdx.x;
  if (threadIdx.x != 0) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int s = 0; s < n_slabs; ++s) {
    const float v = pval[row * n_slabs + s];
    const int i = pidx[row * n_slabs + s];
    if (argmax_better(v, i, best, bi)) { best = v; bi = i; }
  }
  const float first = logits[static_cast<size_t>(row) * V];
  if (first != first || bi == 0x7fffffff) bi = 0;   // NaN in column 0, or no number in the row
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

static bool g_pdl = false;

// Launch with (or without) the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
static cudaError_t launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = g_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Switches programmatic dependent launch of the decode-path kernels (GEMV, RoPE+append,
// flash-decode) on or off for this process; off by default.
extern "C" int sb_set_pdl(int on) { g_pdl = on != 0; return 0; }

namespace sb {
int make_tmap_2d_u16_plain(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                           uint32_t box_inner, uint32_t box_outer);   // gemm_tcgen05.cu
}

template <int MB, bool INT8>
static int launch_gemv_mb(const CUtensorMap& tm, const GemvParams& p, dim3 grid, size_t smem, cudaStream_t s) {
  auto kern = gemv_kernel<MB, INT8>;
  static size_t attr = 0;
  if (smem > attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr = smem;
  }
  return launch_dep(kern, grid, dim3(GEMV_THREADS), smem, s, tm, p) == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

template <bool INT8>
static int launch_gemv(const GemvParams& p, int splits, cudaStream_t s) {
  constexpr int COLS = INT8 ? 512 : 256;
  dim3 grid((p.N + COLS - 1) / COLS, splits);
  const int mb = p.M <= 1 ? 1 : p.M <= 2 ? 2 : p.M <= 4 ? 4 : 8;
  const size_t xs_bytes = static_cast<size_t>(p.k_per_split) * mb * sizeof(float);
  if (xs_bytes > static_cast<size_t>(GEMV_MAX_XS_BYTES)) return SB_ERR_ARG;
  // the RMSNorm prologue borrows the X staging area for mb * 8 * 32 partial sums
  const size_t smem = static_cast<size_t>(GEMV_STAGES) * GEMV_TILE_BYTES +
                      (xs_bytes > static_cast<size_t>(mb) * 1024 ? xs_bytes : static_cast<size_t>(mb) * 1024);
  constexpr int ESZ = INT8 ? 1 : 2;
  CUtensorMap tm;
  const int rc = make_tmap_2d_u16_plain(&tm, p.W, static_cast<uint64_t>(p.N) * ESZ / 2, p.K,
                                        static_cast<uint64_t>(p.ldw) * ESZ, GEMV_ROW_BYTES / 2, GEMV_KT);
  if (rc) return rc;
  switch (mb) {
    case 1: return launch_gemv_mb<1, INT8>(tm, p, grid, smem, s);
    case 2: return launch_gemv_mb<2, INT8>(tm, p, grid, smem, s);
    case 4: return launch_gemv_mb<4, INT8>(tm, p, grid, smem, s);
    default: return launch_gemv_mb<8, INT8>(tm, p, grid, smem, s);
  }
}

namespace sb {
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);   // gemm_tcgen05.cu (128-byte swizzle)
}

// bf16 weights: the tensor-core kernel. The staged slice of X takes 16 bytes per k for every 8 rows.
template <int MBLK>
static int launch_gemv_mma_mb(const GemvParams& p, int splits, cudaStream_t s) {
  dim3 grid((p.N + 255) / 256, splits);
  const int kn_pad = (p.k_per_split + GEMV_KT - 1) / GEMV_KT * GEMV_KT;
  const size_t xs_bytes = static_cast<size_t>(kn_pad) * 16 * MBLK;
  if (xs_bytes > static_cast<size_t>(GEMV_MAX_XS_BYTES)) return SB_ERR_ARG;
  // the RMSNorm prologue borrows the X staging area for M * 8 * 32 partial sums; 1 KB for the ring's alignment
  const size_t borrow = static_cast<size_t>(8 * MBLK) * 1024;
  const size_t smem = static_cast<size_t>(GEMV_STAGES) * GEMV_TILE_BYTES + (xs_bytes > borrow ? xs_bytes : borrow) + 1024;
  CUtensorMap tm;
  const int rc = make_tmap_2d_bf16(&tm, p.W, static_cast<uint64_t>(p.N), p.K, static_cast<uint64_t>(p.ldw), 64, GEMV_KT);
  if (rc) return rc;
  auto kern = gemv_mma_kernel<MBLK>;
  static size_t attr = 0;
  if (smem > attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr = smem;
  }
  return launch_dep(kern, grid, dim3(GEMV_THREADS), smem, s, tm, p) == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
// int8 weights on the tensor-core kernel: the tensor map is over 16-bit words (two int8 columns each).
static int launch_gemv_mma_i8(const GemvParams& p, int splits, cudaStream_t s) {
  dim3 grid((p.N + 511) / 512, splits);
  const int kn_pad = (p.k_per_split + GEMV_KT - 1) / GEMV_KT * GEMV_KT;
  const size_t xs_bytes = static_cast<size_t>(kn_pad) * 16;
  if (xs_bytes > static_cast<size_t>(GEMV_MAX_XS_BYTES)) return SB_ERR_ARG;
  const size_t smem = static_cast<size_t>(GEMV_STAGES) * GEMV_TILE_BYTES + (xs_bytes > 8192 ? xs_bytes : 8192) + 1024;
  if ((p.N & 1) || (p.ldw & 1)) return SB_ERR_ARG;
  CUtensorMap tm;
  const int rc = make_tmap_2d_bf16(&tm, p.W, static_cast<uint64_t>(p.N) / 2, p.K, static_cast<uint64_t>(p.ldw) / 2, 64, GEMV_KT);
  if (rc) return rc;
  auto kern = gemv_mma_i8_kernel;
  static size_t attr = 0;
  if (smem > attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr = smem;
  }
  return launch_dep(kern, grid, dim3(GEMV_THREADS), smem, s, tm, p) == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// Only one block of 8 rows is shipped: with two or four blocks the kernel is bound by the mma.sync rate, not by
// memory (117 MB of weights: 33 us at 8 rows, 58 us at 16, 111 us at 32), and the tcgen05 GEMM is faster there.
static int launch_gemv_mma(const GemvParams& p, int splits, cudaStream_t s) {
  return launch_gemv_mma_mb<1>(p, splits, s);
}

// Y[M,N] = f(X)[M,K] * W[K,N] (* scale[n]) (+ R). M <= 8 per call (callers loop over row groups).
// W bf16 (is_int8 == 0) or int8 with fp32 column scales; the weight row pitch and base must be
// multiples of 16 bytes. workspace: 4096 counter words (zero before the first call, left zero by
// every call) followed by splits*M*N floats. The staged slice of X, (K / splits) * {1,2,4,8} floats,
// must fit in 64 KB: callers raise `splits` accordingly.
// prologue: 0 none, 1 RMSNorm of X with gain norm_w (K must be a multiple of 8), 2 SwiGLU over a
// fused [gate | up] X of row width 2K.
struct GemvCollArgs {
  void* const* recv_ptrs; void* const* flag_ptrs; uint32_t* epoch_word; unsigned int* done_ctr;
  int rank, W, rows, wait_ms;
};

struct GemvAmaxArgs {
  int32_t* ws;                 // word 0: CTA counter (zero between calls); 16...: pval [8][4096]; then pidx [8][4096]
  int64_t* out_tokens; int64_t* generated; int gen_stride, step, col_offset;
  void* const* cand_ptrs; void* const* flag_ptrs; uint32_t* epoch_word; int rank, W, wait_ms;
};

static int gemv_impl(const void* X, int ldx, const void* W, int ldw, const float* scale, const void* R, int ldr,
                     void* out_bf16, int ldo, float* out_f32, int M, int N, int K, int is_int8, int splits,
                     float* workspace, int prologue, const void* norm_w, float eps, int* status, void* stream,
                     const GemvCollArgs* ca, const GemvAmaxArgs* aa = nullptr) {
  if (M <= 0 || M > 8 || N <= 0 || K <= 0 || (N & 7) || (is_int8 && (N & 15))) return SB_ERR_ARG;
  if (prologue < 0 || prologue > 2 || (prologue == 1 && (!norm_w || (K & 7) || (ldx & 7)))) return SB_ERR_ARG;
  const int esz = is_int8 ? 1 : 2;
  if ((reinterpret_cast<uintptr_t>(W) & 15) || ((static_cast<size_t>(ldw) * esz) & 15)) return SB_ERR_ALIGN;
  if (splits < 1) splits = 1;
  // the tensor-core kernels (SB_GEMV_FMA=1 in the environment selects the FMA kernels instead):
  // its k ranges are whole 32-row tiles and its staged X takes 16 bytes per k, so at most 4096 k per split
  static const bool bf16_fma = [] { const char* e = getenv("SB_GEMV_FMA"); return e && e[0] == '1'; }();
  const bool mma = !bf16_fma;   // both weight types take the tensor-core kernels unless the FMA kernels are asked for
  int kps = !mma ? ((K + splits - 1) / splits + 7) / 8 * 8 : ((K + splits - 1) / splits + 31) / 32 * 32;
  if (mma && kps > 4096) kps = 4096;
  splits = (K + kps - 1) / kps;
  const int cols = is_int8 ? 512 : 256;
  if ((N + cols - 1) / cols > 4096) return SB_ERR_ARG;
  GemvParams p;
  p.X = static_cast<const __nv_bfloat16*>(X); p.ldx = ldx; p.W = W; p.ldw = ldw; p.scale = is_int8 ? scale : nullptr;
  p.R = static_cast<const __nv_bfloat16*>(R); p.ldr = ldr;
  p.out = static_cast<__nv_bfloat16*>(out_bf16); p.ldo = ldo; p.out_f32 = out_f32;
  p.counters = reinterpret_cast<unsigned int*>(workspace);
  p.part = workspace + 4096;
  p.M = M; p.N = N; p.K = K; p.k_per_split = kps; p.prologue = prologue;
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w); p.eps = eps; p.status = status;
  p.coll.W = 0; p.coll.rank = 0; p.coll.rows = 0; p.coll.epoch_word = nullptr; p.coll.done_ctr = nullptr;
  p.coll.wait_ns = 0;
  if (ca) {
    if (!mma || ca->W < 2 || ca->W > MAX_WORLD || ca->rank < 0 || ca->rank >= ca->W || ca->rows < M ||
        !ca->epoch_word || !ca->done_ctr || !status)
      return SB_ERR_ARG;
    p.coll.W = ca->W; p.coll.rank = ca->rank; p.coll.rows = ca->rows;
    for (int r = 0; r < ca->W; ++r) {
      if (!ca->recv_ptrs[r] || !ca->flag_ptrs[r]) return SB_ERR_ARG;
      p.coll.recv[r] = static_cast<float*>(ca->recv_ptrs[r]);
      p.coll.flags[r] = static_cast<uint32_t*>(ca->flag_ptrs[r]);
    }
    p.coll.epoch_word = ca->epoch_word; p.coll.done_ctr = ca->done_ctr;
    p.coll.wait_ns = ca->wait_ms > 0 ? static_cast<uint64_t>(ca->wait_ms) * 1000000ull : kPeerWaitNsDefault;
  }
  p.amax.out_tokens = nullptr; p.amax.W = 0;
  if (aa) {
    if (!mma || ca || !aa->ws || !aa->out_tokens || aa->col_offset < 0) return SB_ERR_ARG;
    p.amax.ctr = reinterpret_cast<unsigned int*>(aa->ws);
    p.amax.pval = reinterpret_cast<float*>(aa->ws + 16);
    p.amax.pidx = aa->ws + 16 + 8 * 4096;
    p.amax.out_tokens = aa->out_tokens; p.amax.generated = aa->generated; p.amax.gen_stride = aa->gen_stride;
    p.amax.step = aa->step; p.amax.col_offset = aa->col_offset; p.amax.W = aa->W > 1 ? aa->W : 0;
    p.amax.rank = aa->rank; p.amax.epoch_word = aa->epoch_word;
    p.amax.wait_ns = aa->wait_ms > 0 ? static_cast<uint64_t>(aa->wait_ms) * 1000000ull : kPeerWaitNsDefault;
    if (aa->W > 1) {
      if (aa->W > MAX_WORLD || aa->rank < 0 || aa->rank >= aa->W || !aa->cand_ptrs || !aa->flag_ptrs ||
          !aa->epoch_word || !status)
        return SB_ERR_ARG;
      for (int r = 0; r < aa->W; ++r) {
        if (!aa->cand_ptrs[r] || !aa->flag_ptrs[r]) return SB_ERR_ARG;
        p.amax.cand[r] = static_cast<unsigned long long*>(aa->cand_ptrs[r]);
        p.amax.flags[r] = static_cast<uint32_t*>(aa->flag_ptrs[r]);
      }
    }
  }
  if (mma) return is_int8 ? launch_gemv_mma_i8(p, splits, STREAM) : launch_gemv_mma(p, splits, STREAM);
  return is_int8 ? launch_gemv<true>(p, splits, STREAM) : launch_gemv<false>(p, splits, STREAM);
}

extern "C" int sb_gemv(const void* X, int ldx, const void* W, int ldw, const float* scale, const void* R, int ldr,
                       void* out_bf16, int ldo, float* out_f32, int M, int N, int K, int is_int8, int splits,
                       float* workspace, int prologue, const void* norm_w, float eps, int* status, void* stream) {
  return gemv_impl(X, ldx, W, ldw, scale, R, ldr, out_bf16, ldo, out_f32, M, N, K, is_int8, splits, workspace,
                   prologue, norm_w, eps, status, stream, nullptr);
}

// The row-parallel GEMV of tensor-parallel decoding fused with its all-reduce: out = R + sum over ranks of
// f(X_r) W_r, one launch. recv_ptrs[r]: rank r's receive buffer (peer-mapped, fp32 [2][world][rows][N], rows >= M);
// flag_ptrs[r]: rank r's epoch words [ceil(N / 256 or 512)][16], zero when the channel is created; epoch_word and
// done_ctr: local device words, zero when the channel is created. Every rank must issue the same sequence of
// calls on a channel. Tensor-core kernels only (not with SB_GEMV_FMA=1).
extern "C" int sb_gemv_allreduce(const void* X, int ldx, const void* W, int ldw, const float* scale, const void* R,
                                 int ldr, void* out_bf16, int ldo, int M, int N, int K, int is_int8, int splits,
                                 float* workspace, int prologue, const void* norm_w, float eps,
                                 void* const* recv_ptrs, void* const* flag_ptrs, uint32_t* epoch_word,
                                 unsigned int* done_ctr, int rank, int world, int rows, int wait_ms, int* status,
                                 void* stream) {
  GemvCollArgs ca{recv_ptrs, flag_ptrs, epoch_word, done_ctr, rank, world, rows, wait_ms};
  return gemv_impl(X, ldx, W, ldw, scale, R, ldr, out_bf16, ldo, nullptr, M, N, K, is_int8, splits, workspace,
                   prologue, norm_w, eps, status, stream, &ca);
}

// LM head and greedy arg-max in one launch: out_tokens[m] = argmax over n of (f(X) W)[m, n] + col_offset (NaN in
// global column 0 -> token 0; other NaNs skipped; ties -> lower column). logits_f32 [M, N] is optional. amax_ws:
// 16 + 2 * 8 * 4096 32-bit words, the first one zero before the first call. world > 1: the head is sharded over the
// vocabulary; cand_ptrs[r] / flag_ptrs[r] are rank r's peer-mapped candidate slots (2 * world * 8 64-bit words, zero at
// creation) and epoch words (16), epoch_word a local device word (zero at creation); every rank issues the same calls.
extern "C" int sb_gemv_argmax(const void* X, int ldx, const void* W, int ldw, const float* scale, float* logits_f32,
                              int M, int N, int K, int is_int8, int splits, float* workspace, int prologue,
                              const void* norm_w, float eps, int32_t* amax_ws, int64_t* out_tokens,
                              int64_t* generated, int gen_stride, int step, int col_offset, void* const* cand_ptrs,
                              void* const* flag_ptrs, uint32_t* epoch_word, int rank, int world, int wait_ms,
                              int* status, void* stream) {
  GemvAmaxArgs aa{amax_ws, out_tokens, generated, gen_stride, step, col_offset, cand_ptrs, flag_ptrs, epoch_word,
                  rank, world, wait_ms};
  return gemv_impl(X, ldx, W, ldw, scale, nullptr, 0, nullptr, 0, logits_f32, M, N, K, is_int8, splits, workspace,
                   prologue, norm_w, eps, status, stream, nullptr, &aa);
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
  return launch_dep(rope_kv_append_kernel, dim3(n_tok, H + 2 * Hkv), dim3(dh / 2), 0, STREAM, static_cast<__nv_bfloat16*>(qkv), ld, H,
                    Hkv, dh, cos_t, sin_t, static_cast<__nv_bfloat16*>(pool), block_table, max_blocks, page, seq_of,
                    pos, n_tok) == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// q: bf16 [B, ldq] (H*dh used, RoPE'd); out: bf16 [B, ldo]. part_o: B*H*n_splits*dh floats,
// part_ml: B*H*n_splits*2 floats (scratch).
template <int DH>
static int launch_decode_attn(const DecodeAttnParams& p, dim3 grid, cudaStream_t s) {
  constexpr int SMEM = 2 * 2 * DEC_TK * (DH * 2 + 16);   // also covers the merge buffers (4*16*(DH+2) floats)
  static_assert(SMEM >= 4 * 16 * (DH + 2) * 4, "merge buffers must fit in the tile ring");
  auto kern = decode_attn_kernel<DH>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return SB_ERR_LAUNCH;
    attr = true;
  }
  return launch_dep(kern, grid, dim3(128), SMEM, s, p) == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// q: [B, >= H*dh] bf16 (RoPE'd), out: [B, H*dh] bf16. part_o: B*H*n_splits*dh floats, part_ml:
// B*H*n_splits*2 floats, counters: B*Hkv words that are zero before the first call (every call leaves
// them zero). H / Hkv <= 16, dh in {64, 128}.
extern "C" int sb_decode_attention(const void* q, int ldq, const void* pool, const int* block_table, int max_blocks,
                                   int page, const int* seq_len, int B, int H, int Hkv, int dh, int n_splits,
                                   float scale, float* part_o, float* part_ml, unsigned int* counters, void* out,
                                   int ldo, void* stream) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) || H / Hkv > 16 || (dh != 64 && dh != 128) || n_splits < 1 ||
      page < 1 || (ldq & 1))
    return SB_ERR_ARG;
  DecodeAttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.ldq = ldq;
  p.pool = static_cast<const __nv_bfloat16*>(pool);
  p.block_table = block_table; p.max_blocks = max_blocks; p.page = page; p.seq_len = seq_len;
  p.H = H; p.Hkv = Hkv; p.n_splits = n_splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.part_o = part_o; p.part_ml = part_ml;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.counters = counters;
  dim3 grid(Hkv, B, n_splits);
  return dh == 64 ? launch_decode_attn<64>(p, grid, STREAM) : launch_decode_attn<128>(p, grid, STREAM);
}

// logits: fp32 [rows, V]. pval/pidx: rows * ceil(V/4096) scratch. out_tokens: int64 [rows].
extern "C" int sb_argmax(const float* logits, int rows, int V, float* pval, int* pidx, int64_t* out_tokens,
                         int64_t* generated, int gen_stride, int step, void* stream) {
  if (rows <= 0 || V <= 0) return SB_ERR_ARG;
  const int cpc = 4096;
  const int slabs = (V + cpc - 1) / cpc;
  argmax_partial_kernel<<<dim3(slabs, rows), 256, 0, STREAM>>>(logits, V, cpc, pval, pidx);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  argmax_final_kernel<<<rows, 32, 0, STREAM>>>(logits, V, pval, pidx, slabs, out_tokens, generated, gen_stride, step);
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
