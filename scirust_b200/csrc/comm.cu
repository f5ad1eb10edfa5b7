// Peer-memory substrate and the fused data-parallel gradient all-reduce.
//
// Symmetric memory: every rank cudaMalloc's a region of the same size, exports it with
// cudaIpcGetMemHandle, and maps every peer's region (cudaIpcOpenMemHandle). Kernels then receive
// a table of W base pointers and address a peer's copy of a buffer directly over NVLink.
//
// Flag protocol (all waits bounded; a wait that runs out stores ST_TIMEOUT_PEER in the status
// word and the kernel leaves without touching peer memory again):
//   flags live in each rank's own region: flags[slot][phase][src_rank] (uint32 epochs).
//   A rank announces phase p of call `epoch` by storing `epoch` into flags[slot][p][my_rank] of
//   EVERY peer (st.release.sys) and waits for its own flags[slot][p][*] to reach `epoch`
//   (ld.acquire.sys).
//
// sb_allreduce_bf16 (the data-parallel gradient reduction; reference semantics: rank-ordered sum
// then one multiply by 1/world, scirust-core/src/distributed.rs:96-167). Reads only, no peer stores:
//   phase 0   "my bucket is final"            -> every CTA waits for all peers (W lanes poll W flags)
//   reduce    rank r owns shard r of the bucket: pulls that shard from every rank's bucket with
//             peer loads, adds in rank order 0..W-1 in fp32 (bf16 -> fp32 cast fused), scales by
//             1/W (or any factor), rounds once, and writes the result into shard r of its OWN output
//   phase 1   the last CTA of the rank to finish its part announces "shard r of my output is reduced
//             and I no longer read your bucket"; every CTA waits for all peers
//   gather    pulls the W-1 other reduced shards from the peers' outputs into the local output
//             (bf16 or fp32), eight 16-byte loads in flight per thread
// No closing wait is needed: a peer overwrites its bucket only after its own kernel has passed
// phase 1 (all ranks finished reading buckets), and it overwrites its output shard only in a later
// call, after that call's phase 0, which every rank announces only once this kernel has ended on
// its stream. Because each element is reduced by exactly one rank and copied, all replicas receive
// identical bits, and the sum order is fixed: the result is bitwise repeatable at a fixed world.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include "api.h"
#include "sm100_ptx.cuh"
#include "peer_sync.cuh"

namespace sb {

struct AllReduceParams {
  PeerTable t;
  int rank, W;
  size_t n;            // elements in the bucket (multiple of 8)
  float scale;
  uint32_t epoch;
  int slot;            // flag slot (bucket index)
  int out_fp32;
  uint64_t wait_ns;
  unsigned int* cta_counter;  // local, zero before the call; reset by the kernel
  int* status;
};

__device__ __forceinline__ void accum8(float* acc, const uint4& v) {
  acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
  acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
}

// U = 16-byte vectors per thread and iteration of the reduce phase; with W ranks U * W peer loads are in flight
// before the first add (the host picks U = 8 / 4 / 2 for W <= 2 / <= 4 / larger, so about sixteen).
template <int U, int RG, int THREADS, int MIN_BLOCKS>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS)
allreduce_bf16_kernel(const __grid_constant__ AllReduceParams p) {
  __shared__ int s_ok;
  const int W = p.W;
  uint32_t* my_flags = p.t.flags[p.rank] + static_cast<size_t>(p.slot) * SLOT_WORDS;
  if (threadIdx.x < 32) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      if (threadIdx.x < W)
        st_release_sys(p.t.flags[threadIdx.x] + static_cast<size_t>(p.slot) * SLOT_WORDS + p.rank, p.epoch);
    }
    const bool w = wait_flags_warp(my_flags, W, p.epoch, p.wait_ns, p.status);
    if (threadIdx.x == 0) s_ok = w ? 1 : 0;
  }
  __syncthreads();
  bool ok = s_ok != 0;
  // shard r = [r*per, min(n, (r+1)*per)), per a multiple of 8 elements
  const size_t per = ((p.n + W - 1) / W + 7) / 8 * 8;
  const size_t gtid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;

  if (ok) {
    const size_t lo = min(p.n, per * p.rank);
    const size_t hi = min(p.n, lo + per);
    const size_t n8 = (hi - lo) / 8;
    for (size_t i0 = gtid; i0 < n8; i0 += U * stride) {
      float accs[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) accs[u][j] = 0.f;
      for (int r0 = 0; r0 < W; r0 += RG) {     // ranks in groups: loads first, then the adds in rank order
        uint4 v[RG][U];
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          if (r0 + r < W) {
            const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(p.t.in[r0 + r]) + lo;
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (i0 + u * stride < n8) v[r][u] = ld_peer_v4(base + (i0 + u * stride) * 8);
          }
        }
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          if (r0 + r < W) {
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (i0 + u * stride < n8) accum8(accs[u], v[r][u]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * stride >= n8) break;
        const size_t e = lo + (i0 + u * stride) * 8;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = accs[u][j] * p.scale;
        if (p.out_fp32) {
          float* o = static_cast<float*>(p.t.out[p.rank]) + e;
          *reinterpret_cast<uint4*>(o) = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]),
                                                    __float_as_uint(acc[2]), __float_as_uint(acc[3]));
          *reinterpret_cast<uint4*>(o + 4) = make_uint4(__float_as_uint(acc[4]), __float_as_uint(acc[5]),
                                                        __float_as_uint(acc[6]), __float_as_uint(acc[7]));
        } else {
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.t.out[p.rank]) + e) =
              make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                         pack_bf16x2(acc[6], acc[7]));
        }
      }
    }
  }
  // the last CTA of this rank to finish its part of the shard tells every peer that the shard is reduced
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned int prev = 0;
    if (threadIdx.x == 0) prev = atomicAdd(p.cta_counter, 1u);
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if (prev == gridDim.x - 1) {
      if (threadIdx.x == 0) *p.cta_counter = 0;  // ready for the next call on this stream
      if (ok) {
        __threadfence_system();
        if (threadIdx.x < W)
          st_release_sys(p.t.flags[threadIdx.x] + static_cast<size_t>(p.slot) * SLOT_WORDS + MAX_WORLD + p.rank,
                         p.epoch);
      }
    }
    if (ok) {
      const bool w = wait_flags_warp(my_flags + MAX_WORLD, W, p.epoch, p.wait_ns, p.status);
      if (threadIdx.x == 0) s_ok = w ? 1 : 0;
    }
  }
  __syncthreads();
  ok = ok && s_ok != 0;
  if (!ok) return;

  // gather: copy the other ranks' reduced shards, 16-byte words, eight loads in flight per thread
  const size_t esz = p.out_fp32 ? 4 : 2;
  uint4* mine = static_cast<uint4*>(p.t.out[p.rank]);
  for (int q0 = 1; q0 < W; ++q0) {
    const int q = (p.rank + q0) % W;          // start with the next rank so the peers' links are spread
    const size_t lo = min(p.n, per * q), hi = min(p.n, lo + per);
    const size_t w0 = lo * esz / 16, nw = (hi - lo) * esz / 16;
    const uint4* src = static_cast<const uint4*>(p.t.out[q]) + w0;
    uint4* dst = mine + w0;
    for (size_t i = gtid; i < nw; i += 8 * stride) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i + u * stride < nw) v[u] = ld_peer_v4(src + i + u * stride);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i + u * stride < nw) dst[i + u * stride] = v[u];
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Latency-oriented collectives for tensor-parallel decoding (messages of a few KB to a few hundred
// KB). One wait per call instead of two, output in plain local memory, and the epoch lives in a
// device word that the kernel itself advances, so a captured CUDA graph can replay the call.
//
//   every rank: source buffer (its partial result, symmetric memory) is final when the kernel starts
//   announce  flags[slot][0][my_rank] = epoch on every peer; wait for all peers' announcements
//   mode 0    out[i] = residual[i] + sum over ranks r = 0..W-1 of in[r][i]   (fp32, fixed order, so
//             every rank computes identical bits; inputs bf16 or fp32, output bf16)
//   mode 1    out[row][r][i] = in[r][row][i]   (all-gather of 16-byte words, e.g. vocabulary-
//             sharded logits rows)
// There is no closing wait: a source buffer may be rewritten only after the same rank has completed
// a LATER collective on this channel (every peer entered that later call, hence finished reading).
// Callers alternate at least two source buffers per channel.
struct SmallCollParams {
  const void* in[MAX_WORLD];
  uint32_t* flags[MAX_WORLD];
  int rank, W, mode, in_fp32;
  size_t n;          // mode 0: elements (multiple of 8); mode 1: 16-byte words per row per rank
  int rows;          // mode 1
  const __nv_bfloat16* residual;  // mode 0, may be null
  void* out;
  uint32_t* epoch_word;       // local device word: number of completed calls on this channel
  int slot;
  uint64_t wait_ns;
  unsigned int* cta_counter;
  int* status;
};

__global__ void __launch_bounds__(256)
small_collective_kernel(const __grid_constant__ SmallCollParams p) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  const int W = p.W;
  if (threadIdx.x == 0) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.epoch_word) + 1u;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < W; ++r)
        st_release_sys(p.flags[r] + static_cast<size_t>(p.slot) * SLOT_WORDS + p.rank, e);
    }
    s_ok = wait_flags(p.flags[p.rank] + static_cast<size_t>(p.slot) * SLOT_WORDS, W, e, p.wait_ns, p.status) ? 1 : 0;
    s_epoch = e;
  }
  __syncthreads();
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (s_ok) {
    if (p.mode == 0) {
      const size_t n8 = p.n / 8;
      for (size_t i = tid; i < n8; i += nthreads) {
        float acc[8];
        if (p.residual) {
          const uint4 v = *reinterpret_cast<const uint4*>(p.residual + i * 8);
          acc[0] = bf16_lo(v.x); acc[1] = bf16_hi(v.x); acc[2] = bf16_lo(v.y); acc[3] = bf16_hi(v.y);
          acc[4] = bf16_lo(v.z); acc[5] = bf16_hi(v.z); acc[6] = bf16_lo(v.w); acc[7] = bf16_hi(v.w);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
        for (int r = 0; r < W; ++r) {
          if (p.in_fp32) {
            const float* src = static_cast<const float*>(p.in[r]) + i * 8;
            const uint4 a = ld_peer_v4(src), b = ld_peer_v4(src + 4);
            acc[0] += __uint_as_float(a.x); acc[1] += __uint_as_float(a.y);
            acc[2] += __uint_as_float(a.z); acc[3] += __uint_as_float(a.w);
            acc[4] += __uint_as_float(b.x); acc[5] += __uint_as_float(b.y);
            acc[6] += __uint_as_float(b.z); acc[7] += __uint_as_float(b.w);
          } else {
            const uint4 v = ld_peer_v4(static_cast<const __nv_bfloat16*>(p.in[r]) + i * 8);
            acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
            acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
          }
        }
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + i * 8) =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                       pack_bf16x2(acc[6], acc[7]));
      }
    } else {
      const size_t per_rank = static_cast<size_t>(p.rows) * p.n;
      const size_t total = per_rank * W;
      uint4* out = static_cast<uint4*>(p.out);
      for (size_t i = tid; i < total; i += nthreads) {
        const int r = static_cast<int>(i / per_rank);
        const size_t w = i - static_cast<size_t>(r) * per_rank;
        const size_t row = w / p.n, col = w - row * p.n;
        out[(row * W + r) * p.n + col] = ld_peer_v4(static_cast<const uint4*>(p.in[r]) + w);
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.cta_counter = 0;
      *reinterpret_cast<volatile uint32_t*>(p.epoch_word) = s_epoch;
    }
  }
}

// A wait that nothing satisfies: used by tests to check that a bounded wait returns a status
// instead of hanging. Waits `limit_ns` at most on flags that stay below `epoch`.
__global__ void wait_probe_kernel(const uint32_t* flags, int W, uint32_t epoch, uint64_t limit_ns, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_flags(flags, W, epoch, limit_ns, status);
}

}  // namespace sb

using namespace sb;

extern "C" int sb_malloc(size_t bytes, void** out) {
  return cudaMalloc(out, bytes) == cudaSuccess ? 0 : SB_ERR_RUNTIME;
}
extern "C" int sb_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : SB_ERR_RUNTIME; }
extern "C" int sb_memset(void* p, int v, size_t bytes, void* stream) {
  return cudaMemsetAsync(p, v, bytes, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : SB_ERR_RUNTIME;
}
// handle_out: 64 bytes
extern "C" int sb_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return SB_ERR_RUNTIME;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int sb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : SB_ERR_RUNTIME;
}
extern "C" int sb_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : SB_ERR_RUNTIME; }
extern "C" int sb_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
extern "C" int sb_flag_words_per_slot() { return SLOT_WORDS; }

// in_ptrs/out_ptrs/flag_ptrs: host arrays of W device pointers (peer-mapped; entry `rank` is local).
// n_elems must be a multiple of 8; buffers 16-byte aligned. wait_ms <= 0 selects the default.
static int allreduce_bf16_impl(void* const* in_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int rank,
                               int W, size_t n_elems, float scale, uint32_t epoch, int slot, int out_fp32,
                               unsigned int* cta_counter, int n_ctas, int wait_ms, int* status, void* stream, bool lean) {
  if (W < 1 || W > MAX_WORLD || rank < 0 || rank >= W || (n_elems & 7) || n_ctas < 1) return SB_ERR_ARG;
  if (cta_counter == nullptr || status == nullptr || in_ptrs == nullptr || out_ptrs == nullptr || flag_ptrs == nullptr)
    return SB_ERR_ARG;
  AllReduceParams p;
  for (int r = 0; r < W; ++r) {
    if ((reinterpret_cast<uintptr_t>(in_ptrs[r]) & 15) || (reinterpret_cast<uintptr_t>(out_ptrs[r]) & 15))
      return SB_ERR_ALIGN;
    p.t.in[r] = in_ptrs[r];
    p.t.out[r] = out_ptrs[r];
    p.t.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  p.rank = rank; p.W = W; p.n = n_elems; p.scale = scale; p.epoch = epoch; p.slot = slot;
  p.out_fp32 = out_fp32;
  p.wait_ns = wait_ms > 0 ? static_cast<uint64_t>(wait_ms) * 1000000ull : kPeerWaitNsDefault;
  p.cta_counter = cta_counter;
  p.status = status;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (lean) {
    // 128 threads x 64 registers: a CTA of this shape fits on an SM beside a resident GEMM CTA (448 threads x 128
    // registers), so a bucket reduced on a side stream during backward neither waits for whole SMs to drain nor
    // keeps GEMM CTAs off the SMs it sits on while it waits for its peers
    if (W <= 2) allreduce_bf16_kernel<4, 2, 128, 8><<<n_ctas, 128, 0, st>>>(p);
    else if (W <= 4) allreduce_bf16_kernel<2, 4, 128, 8><<<n_ctas, 128, 0, st>>>(p);
    else allreduce_bf16_kernel<1, 8, 128, 8><<<n_ctas, 128, 0, st>>>(p);
  } else {
    // sixteen vectors per thread; eight per rank need more than the 128 registers a 512-thread block leaves:
    // half-size blocks, twice as many
    if (W <= 2) allreduce_bf16_kernel<8, 2, 256, 1><<<2 * n_ctas, 256, 0, st>>>(p);
    else if (W <= 4) allreduce_bf16_kernel<4, 4, 512, 1><<<n_ctas, 512, 0, st>>>(p);
    else allreduce_bf16_kernel<2, 8, 512, 1><<<n_ctas, 512, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_allreduce_bf16(void* const* in_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int rank,
                                 int W, size_t n_elems, float scale, uint32_t epoch, int slot, int out_fp32,
                                 unsigned int* cta_counter, int n_ctas, int wait_ms, int* status, void* stream) {
  return allreduce_bf16_impl(in_ptrs, out_ptrs, flag_ptrs, rank, W, n_elems, scale, epoch, slot, out_fp32, cta_counter,
                             n_ctas, wait_ms, status, stream, false);
}
// Same collective, same bits, in CTAs of 128 threads x 64 registers for calls that overlap other kernels.
extern "C" int sb_allreduce_bf16_lean(void* const* in_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int rank,
                                      int W, size_t n_elems, float scale, uint32_t epoch, int slot, int out_fp32,
                                      unsigned int* cta_counter, int n_ctas, int wait_ms, int* status, void* stream) {
  return allreduce_bf16_impl(in_ptrs, out_ptrs, flag_ptrs, rank, W, n_elems, scale, epoch, slot, out_fp32, cta_counter,
                             n_ctas, wait_ms, status, stream, true);
}

// mode 0: all-reduce sum (+ residual) of n elements -> bf16 `out` (local memory);
// mode 1: all-gather of `rows` rows of n 16-byte words per rank -> out[row][rank][n].
// epoch_word and cta_counter are local device words, zero when the channel is created.
extern "C" int sb_small_collective(void* const* in_ptrs, void* const* flag_ptrs, int rank, int W, int mode,
                                   int in_fp32, size_t n, int rows, const void* residual, void* out,
                                   uint32_t* epoch_word, int slot, unsigned int* cta_counter, int n_ctas, int wait_ms,
                                   int* status, void* stream) {
  if (W < 1 || W > MAX_WORLD || rank < 0 || rank >= W || n_ctas < 1 || mode < 0 || mode > 1) return SB_ERR_ARG;
  if (mode == 0 && (n & 7)) return SB_ERR_ARG;
  if (mode == 1 && rows < 1) return SB_ERR_ARG;
  if (cta_counter == nullptr || status == nullptr || epoch_word == nullptr || out == nullptr) return SB_ERR_ARG;
  SmallCollParams p;
  for (int r = 0; r < W; ++r) {
    if (reinterpret_cast<uintptr_t>(in_ptrs[r]) & 15) return SB_ERR_ALIGN;
    p.in[r] = in_ptrs[r];
    p.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15)) return SB_ERR_ALIGN;
  p.rank = rank; p.W = W; p.mode = mode; p.in_fp32 = in_fp32; p.n = n; p.rows = rows;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = out; p.epoch_word = epoch_word; p.slot = slot;
  p.wait_ns = wait_ms > 0 ? static_cast<uint64_t>(wait_ms) * 1000000ull : kPeerWaitNsDefault;
  p.cta_counter = cta_counter; p.status = status;
  small_collective_kernel<<<n_ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_wait_probe(const void* flags, int W, uint32_t epoch, int wait_ms, int* status, void* stream) {
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(flags), W, epoch, static_cast<uint64_t>(wait_ms) * 1000000ull, status);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
