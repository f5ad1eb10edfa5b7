// Tensor-parallel GEMMs fused with their collective, for sm_100a, over NVLink peer memory.
//
// One kernel family, built on the same TMA -> tcgen05.mma -> TMEM pipeline as gemm_tcgen05.cu:
//
//  * all-gather -> GEMM  (column-parallel QKV and gate/up projections, and every product whose
//    token dimension is sharded over the ranks): rank s holds rows [s*R, (s+1)*R) of the operand.
//    When the sharded rows are the M rows of A (the forward products), four copier warps per CTA
//    pull the peers' shards into a LOCAL staging buffer, 128-row chunk by chunk in the order the
//    tiles will need them, with plain peer loads; a chunk's counter raises its "landed" flag and
//    the TMA producer waits (bounded) for that flag before it loads the chunk's tiles from local
//    memory. So every remote byte crosses NVLink once, while the tensor cores work on the local
//    shard and on chunks that have landed. (Reading each remote tile straight from the peer by
//    TMA, as the other operand forms still do, re-fetches it once per column tile: measured 3.3 ms
//    against 0.8 ms for NCCL all-gather + cuBLAS at 16384 x 4096 x 7168 on two GPUs.)
//    Operands sharded along K (weight-gradient forms) are read tile by tile from the owning rank
//    through per-peer tensor maps (plain TMA loads of peer memory, no multicast).
//  * GEMM -> reduce-scatter  (row-parallel o_proj and down_proj): the epilogue stores each partial
//    output tile as bf16 into the staging slot [src = my rank] of the rank that owns those rows
//    (peer stores); per-owner counters tell when all tiles for an owner have been delivered and a
//    flag is raised on that owner. After its own tiles, every CTA waits (bounded) for the flags
//    of all sources and adds the W slots of its rows in rank order 0..W-1 (+ residual), so the
//    result is bitwise repeatable at a fixed world size. Owners are served in the order
//    rank+1, rank+2, ..., rank, so transfers start with the first tiles and the local rows,
//    which need no transfer, come last.
//
// The reference has no tensor parallelism (it states "no multi-GPU, no NCCL", src/lib.rs:133); the
// reduction-order contract kept here is the one of its host collectives
// (scirust-core/src/distributed.rs:96-167: sum in ascending rank order).
//
// Flags (uint32 epochs, in each rank's own symmetric region, one slot per call site):
//   [0*16 + s] rank s's gathered operand is final ("ready")
//   [1*16 + s] rank s no longer reads my operand ("done")
//   [2*16 + s] rank s has delivered all its partial tiles for my rows ("delivered")
// All waits are bounded; on expiry ST_TIMEOUT_PEER is stored in the status word and the kernel
// stops touching peer memory and falls through to its teardown.
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int num_sms();

constexpr int DBM = 128;
constexpr int DBK = 64;
constexpr int DIST_THREADS = 448;   // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue, warps 10-13 copiers
constexpr int COPY_WARPS = 4;
constexpr int DMAXW = 8;
constexpr int FLAG_STRIDE = 16;

template <int BN>
struct DistCfg {
  static constexpr int A_BYTES = DBM * DBK * 2;
  static constexpr int B_BYTES = BN * DBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

struct DistMaps {
  CUtensorMap a[DMAXW];
  CUtensorMap b[DMAXW];
  CUtensorMap a_stage;       // local staging of the gathered A ([M, K], same box as a[])
};

struct DistParams {
  int M, N, K;
  int W, rank;
  int a_gather, b_gather;    // operand's stored rows are sharded over the ranks
  int rows_a, rows_b;        // stored rows per rank of the gathered operand
  int scatter;               // reduce-scatter the output over M
  void* C; int ldc;          // local output: [M, ldc], or [M/W, ldc] when scatter
  const void* R; int ldr;    // optional residual (same row space as C)
  void* stage[DMAXW];        // scatter: staging base on each rank (already offset by buffer parity)
  uint32_t* flags[DMAXW];    // this call site's flag slot on each rank
  uint32_t epoch;
  unsigned int* counters;    // local, zero on entry: [0] CTAs finished, [1 + o] epilogue warps done for owner o
  uint64_t wait_ns;
  int* status;
  // all-gather staging (A sharded along its M rows): local buffer [M, ld_stage] bf16, per-m-tile
  // "landed" flags (epoch values) and piece counters (zero on entry, reset by the kernel)
  void* a_stage; int ld_stage;
  const void* a_peer[DMAXW]; int lda;
  uint32_t* chunk_flags;
  unsigned int* chunk_ctr;
};

__device__ __forceinline__ void d_st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t d_ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ bool d_wait_flag_gpu(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns, int* status) {
  if (static_cast<int32_t>(d_ld_acquire_gpu(flag) - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(d_ld_acquire_gpu(flag) - epoch) < 0) {
    if ((++spins & 0xff) == 0) {
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, 0, ST_TIMEOUT_PEER);
        return false;
      }
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
    }
  }
  return true;
}

__device__ __forceinline__ void d_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t d_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ bool d_wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns, int* status) {
  if (static_cast<int32_t>(d_ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(d_ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 0xff) == 0) {
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, 0, ST_TIMEOUT_PEER);
        return false;
      }
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
    }
  }
  return true;
}

// Tile order. mode 0: n-major over all m. mode 1 (scatter): all tiles of owner rank+1 first, then
// rank+2, ..., own rows last. mode 2 (operand gathered along M): own rows first, then rank+1, ...
__device__ __forceinline__ void tile_coords(int t, int mt, int nt, int W, int rank, int mode, int& m_idx,
                                            int& n_idx) {
  if (mode == 0) {
    n_idx = t / mt;
    m_idx = t - n_idx * mt;
    return;
  }
  const int mpr = mt / W;  // m tiles per rank
  const int tpr = mpr * nt;
  const int slot = t / tpr;
  const int within = t - slot * tpr;
  n_idx = within / mpr;
  const int m_in = within - n_idx * mpr;
  m_idx = ((slot + rank + (mode == 1 ? 1 : 0)) % W) * mpr + m_in;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(DIST_THREADS, 1)
gemm_dist_kernel(const __grid_constant__ DistMaps maps, const __grid_constant__ DistParams p) {
  using Cfg = DistCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tmem_full = empty_bar + Cfg::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = p.W;
  const int mt = (p.M + DBM - 1) / DBM;
  const int nt = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + DBK - 1) / DBK;
  const int tiles_total = mt * nt;
  const uint32_t* my_flags = p.flags[p.rank];
  const bool gather = p.a_gather || p.b_gather;
  // rotations that put local data first (gather) / local rows last (scatter)
  const bool gather_m = p.a_gather && !A_MN;  // A's stored rows are M
  const bool gather_k = (p.a_gather && A_MN) || p.b_gather;  // stored rows are K
  const int tmode = p.scatter ? 1 : (gather_m ? 2 : 0);
  const int k_rot = gather_k ? p.rank * (num_kb / W) : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 8); }
    fence_barrier_init();
    fence_proxy_async_smem();
    if (gather && blockIdx.x == 0) {
      // my operand shard is final (stream order): tell every peer
      __threadfence_system();
      for (int r = 0; r < W; ++r) d_st_release_sys(p.flags[r] + 0 * FLAG_STRIDE + p.rank, p.epoch);
    }
  }
  if (warp == 1) { tmem_alloc(tmem_holder, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t ready_mask = 1u << p.rank;
      int landed_m = -1;
      auto ensure = [&](int src) -> bool {
        if (ready_mask & (1u << src)) return true;
        if (!d_wait_flag(my_flags + 0 * FLAG_STRIDE + src, p.epoch, p.wait_ns, p.status)) return false;
        ready_mask |= 1u << src;
        return true;
      };
      for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(t, mt, nt, W, p.rank, tmode, m_idx, n_idx);
        for (int kk = 0; kk < num_kb && ok; ++kk) {
          const int kb = (kk + k_rot) % num_kb;
          // source rank and local coordinates of this stage's A and B tiles
          int a_src = p.rank, a_row = A_MN ? kb * DBK : m_idx * DBM;
          if (p.a_gather) { a_src = a_row / p.rows_a; a_row -= a_src * p.rows_a; }
          int b_src = p.rank, b_row = B_MN ? kb * DBK : n_idx * BN;
          if (p.b_gather) { b_src = b_row / p.rows_b; b_row -= b_src * p.rows_b; }
          const bool staged = !A_MN && p.a_stage != nullptr && a_src != p.rank;
          if (staged) {
            // the chunk must have landed in the local staging buffer (copier warps of all CTAs)
            if (landed_m != m_idx) {
              if (!d_wait_flag_gpu(p.chunk_flags + m_idx, p.epoch, p.wait_ns, p.status)) { ok = false; break; }
              asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy stores -> TMA reads
              landed_m = m_idx;
            }
          } else if (!ensure(a_src)) { ok = false; break; }
          if (!ensure(b_src)) { ok = false; break; }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb_ = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          if constexpr (!A_MN) {
            if (staged) tma_load_2d(sa, &maps.a_stage, &full_bar[stage], kb * DBK, m_idx * DBM);
            else tma_load_2d(sa, &maps.a[a_src], &full_bar[stage], kb * DBK, a_row);
          } else {
#pragma unroll
            for (int c = 0; c < DBM / 64; ++c)
              tma_load_2d(sa + c * (64 * DBK * 2), &maps.a[a_src], &full_bar[stage], m_idx * DBM + c * 64, a_row);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb_, &maps.b[b_src], &full_bar[stage], kb * DBK, b_row);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb_ + c * (64 * DBK * 2), &maps.b[b_src], &full_bar[stage], n_idx * BN + c * 64, b_row);
          }
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(DBM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kk = 0; kk < num_kb; ++kk) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t sb_ = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < DBK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * (16 * 128), 64 * DBK * 2, 1024)
                                        : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb_ + k * (16 * 128), 64 * DBK * 2, 1024)
                                        : make_smem_desc(sb_ + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kk > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else if (warp >= 10) {
    // -------------------------------- copiers ---------------------------------
    // Pull the peers' shards of A into local staging, one 128-row chunk at a time in the order the
    // tiles need them (rank+1's rows first); every CTA copies its slice of every chunk, so a chunk
    // lands as early as the link allows.
    if (!A_MN && p.a_stage != nullptr && p.a_gather) {
      const int cw = warp - 10;
      const int mpr = mt / W;
      const size_t vec_per_row = static_cast<size_t>(p.K) / 8;             // 16-byte words per row
      const size_t vec_per_chunk = vec_per_row * DBM;
      const size_t lo = vec_per_chunk * blockIdx.x / gridDim.x, hi = vec_per_chunk * (blockIdx.x + 1) / gridDim.x;
      bool ok = true;
      for (int s = 1; s < W && ok; ++s) {
        const int src = (p.rank + s) % W;
        int ready = 1;
        if (lane == 0) ready = d_wait_flag(my_flags + 0 * FLAG_STRIDE + src, p.epoch, p.wait_ns, p.status) ? 1 : 0;
        ready = __shfl_sync(0xffffffffu, ready, 0);
        if (!ready) break;
        const uint4* peer = static_cast<const uint4*>(p.a_peer[src]);
        for (int mi = 0; mi < mpr; ++mi) {
          const int m_idx = src * mpr + mi;
          const size_t prow0 = static_cast<size_t>(mi) * DBM, srow0 = static_cast<size_t>(m_idx) * DBM;
          for (size_t v0 = lo + (cw * 32 + lane); v0 < hi; v0 += COPY_WARPS * 32 * 4) {
            uint4 tmp[4];
            size_t idx[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              idx[u] = v0 + static_cast<size_t>(u) * COPY_WARPS * 32;
              if (idx[u] < hi) {
                const size_t r = idx[u] / vec_per_row, c = idx[u] - r * vec_per_row;
                const uint4* src_p = peer + ((prow0 + r) * p.lda) / 8 + c;
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(tmp[u].x), "=r"(tmp[u].y), "=r"(tmp[u].z), "=r"(tmp[u].w) : "l"(src_p) : "memory");
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (idx[u] < hi) {
                const size_t r = idx[u] / vec_per_row, c = idx[u] - r * vec_per_row;
                *(static_cast<uint4*>(p.a_stage) + ((srow0 + r) * p.ld_stage) / 8 + c) = tmp[u];
              }
            }
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) {
            const unsigned int prev = atomicAdd(p.chunk_ctr + m_idx, 1u);
            if (prev + 1 == gridDim.x * COPY_WARPS) d_st_release_gpu(p.chunk_flags + m_idx, p.epoch);
          }
        }
      }
      (void)ok;
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int rows_local = p.scatter ? p.M / W : p.M;
    const int tiles_per_owner = p.scatter ? (mt / W) * nt : 0;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x, ++it) {
      int m_idx, n_idx;
      tile_coords(t, mt, nt, W, p.rank, tmode, m_idx, n_idx);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m_idx * DBM + q * 32 + lane;
      const uint32_t taddr_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      int owner = 0;
      __nv_bfloat16* out_row;
      const __nv_bfloat16* res_row = nullptr;
      if (p.scatter) {
        owner = (m_idx * DBM) / rows_local;
        const int lrow = row - owner * rows_local;
        out_row = static_cast<__nv_bfloat16*>(p.stage[owner]) +
                  (static_cast<size_t>(p.rank) * rows_local + lrow) * static_cast<size_t>(p.N);
      } else {
        out_row = static_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc;
        if (p.R) res_row = static_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr;
      }
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_idx * BN + c * 32;
        if (row < p.M && col0 < p.N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p.N) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              if (res_row) {
                const uint4 rv = *reinterpret_cast<const uint4*>(res_row + col0 + v * 8);
                f[0] += bf16_lo(rv.x); f[1] += bf16_hi(rv.x);
                f[2] += bf16_lo(rv.y); f[3] += bf16_hi(rv.y);
                f[4] += bf16_lo(rv.z); f[5] += bf16_hi(rv.z);
                f[6] += bf16_lo(rv.w); f[7] += bf16_hi(rv.w);
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(out_row + col0 + v * 8) = o;
            }
          }
        }
      }
      tc_fence_before();
      if (p.scatter) {
        // this warp's share of the tile is on its way to `owner`: make it visible system-wide,
        // then count it; the warp that completes the owner's count raises the flag there.
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const unsigned int prev = atomicAdd(p.counters + 1 + owner, 1u);
          if (prev + 1 == static_cast<unsigned int>(tiles_per_owner) * 8u) {
            __threadfence_system();
            d_st_release_sys(p.flags[owner] + 2 * FLAG_STRIDE + p.rank, p.epoch);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }

    if (p.scatter) {
      // ---- reduce my rows: wait for every source, add the W slots in rank order ----
      int all = ok ? 1 : 0;
      if (lane == 0 && ok) {
        for (int s = 0; s < W; ++s)
          if (!d_wait_flag(my_flags + 2 * FLAG_STRIDE + s, p.epoch, p.wait_ns, p.status)) { all = 0; break; }
      }
      all = __shfl_sync(0xffffffffu, all, 0);
      if (all) {
        const __nv_bfloat16* st = static_cast<const __nv_bfloat16*>(p.stage[p.rank]);
        const size_t slot = static_cast<size_t>(rows_local) * p.N;
        const size_t n8 = slot / 8;
        const size_t tid = static_cast<size_t>(blockIdx.x) * 256 + (warp - 2) * 32 + lane;
        for (size_t i = tid; i < n8; i += static_cast<size_t>(gridDim.x) * 256) {
          const size_t e = i * 8;
          float acc8[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc8[j] = 0.f;
          for (int s = 0; s < W; ++s) {
            uint4 v;
            const __nv_bfloat16* src = st + s * slot + e;
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
            acc8[0] += bf16_lo(v.x); acc8[1] += bf16_hi(v.x);
            acc8[2] += bf16_lo(v.y); acc8[3] += bf16_hi(v.y);
            acc8[4] += bf16_lo(v.z); acc8[5] += bf16_hi(v.z);
            acc8[6] += bf16_lo(v.w); acc8[7] += bf16_hi(v.w);
          }
          const size_t lrow = e / p.N;
          const int col = static_cast<int>(e - lrow * p.N);
          if (p.R) {
            const uint4 rv = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.R) + lrow * p.ldr + col);
            acc8[0] += bf16_lo(rv.x); acc8[1] += bf16_hi(rv.x);
            acc8[2] += bf16_lo(rv.y); acc8[3] += bf16_hi(rv.y);
            acc8[4] += bf16_lo(rv.z); acc8[5] += bf16_hi(rv.z);
            acc8[6] += bf16_lo(rv.w); acc8[7] += bf16_hi(rv.w);
          }
          uint4 o;
          o.x = pack_bf16x2(acc8[0], acc8[1]);
          o.y = pack_bf16x2(acc8[2], acc8[3]);
          o.z = pack_bf16x2(acc8[4], acc8[5]);
          o.w = pack_bf16x2(acc8[6], acc8[7]);
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.C) + lrow * p.ldc + col) = o;
        }
      }
    }
  }

  // Teardown. Every loop above is bounded, so all threads arrive here.
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  if (threadIdx.x == 0) {
    // last CTA: reset the counters for the next call; with a gathered operand also tell the peers
    // that this rank has stopped reading them, and stay until they have stopped reading this rank.
    __threadfence();
    const unsigned int prev = atomicAdd(p.counters, 1u);
    if (prev == gridDim.x - 1) {
      for (int i = 0; i <= W; ++i) p.counters[i] = 0;
      if (p.chunk_ctr) for (int i = 0; i < mt; ++i) p.chunk_ctr[i] = 0;
      if (gather && *reinterpret_cast<volatile int*>(p.status) == 0) {
        __threadfence_system();
        for (int r = 0; r < W; ++r) d_st_release_sys(p.flags[r] + 1 * FLAG_STRIDE + p.rank, p.epoch);
        for (int s = 0; s < W; ++s)
          if (!d_wait_flag(my_flags + 1 * FLAG_STRIDE + s, p.epoch, p.wait_ns, p.status)) break;
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN>
static int launch_dist(const DistMaps& maps, const DistParams& p, int grid, cudaStream_t stream) {
  using Cfg = DistCfg<BN>;
  auto kern = gemm_dist_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  kern<<<grid, DIST_THREADS, Cfg::SMEM_BYTES, stream>>>(maps, p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

using namespace sb;

// Distributed GEMM. a_ptrs / b_ptrs: host arrays of W device pointers to each rank's copy of the
// operand (all equal to the local pointer when the operand is not gathered). Operand shapes are the
// *global* logical shapes (M, N, K); a gathered operand's stored rows are split evenly over the
// ranks. scatter != 0: C is [M/W, ldc] and stage_ptrs[o] is rank o's staging base for this call
// (W * (M/W) * N bf16); flag_ptrs[r] is rank r's flag slot (48 words). counters: W+1 zeroed words.
// a_stage (optional, local): [M, ld_stage] bf16 landing buffer for a gathered K-major A, with
// chunk_flags / chunk_ctr of ceil(M/128) words each (counters zero on entry).
extern "C" int sb_gemm_dist_bf16(void* const* a_ptrs, void* const* b_ptrs, void* C, const void* R,
                                 void* const* stage_ptrs, void* const* flag_ptrs, int M, int N, int K, int lda,
                                 int ldb, int ldc, int ldr, int a_mn, int b_mn, int a_gather, int b_gather,
                                 int scatter, int rank, int W, uint32_t epoch, unsigned int* counters, int bn,
                                 int wait_ms, void* a_stage, int ld_stage, uint32_t* chunk_flags,
                                 unsigned int* chunk_ctr, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || W < 1 || W > DMAXW || rank < 0 || rank >= W) return SB_ERR_ARG;
  if ((N & 7) || (ldc & 7) || (R && (ldr & 7))) return SB_ERR_ALIGN;
  if (bn == 0) bn = (N <= 128) ? 128 : 256;
  if (bn != 128 && bn != 256) return SB_ERR_ARG;
  if (b_gather && !b_mn) return SB_ERR_ARG;  // only an operand stored [tokens, features] can be sharded by rows
  const int mt = (M + DBM - 1) / DBM, num_kb = (K + DBK - 1) / DBK;
  // shard boundaries must coincide with tile boundaries
  if (scatter && ((M % (W * DBM)) != 0)) return SB_ERR_ARG;
  int rows_a = 0, rows_b = 0;
  if (a_gather) {
    const int total = a_mn ? K : M;
    const int unit = a_mn ? DBK : DBM;
    if (total % (W * unit)) return SB_ERR_ARG;
    rows_a = total / W;
  }
  if (b_gather) {
    if (K % (W * DBK)) return SB_ERR_ARG;
    rows_b = K / W;
  }
  (void)mt; (void)num_kb;

  DistMaps maps;
  for (int r = 0; r < W; ++r) {
    int rc;
    const void* ap = a_ptrs[r];
    const void* bp = b_ptrs[r];
    if (!a_mn) rc = make_tmap_2d_bf16(&maps.a[r], ap, K, a_gather ? rows_a : M, lda, DBK, DBM);
    else rc = make_tmap_2d_bf16(&maps.a[r], ap, M, a_gather ? rows_a : K, lda, 64, DBK);
    if (rc) return rc;
    if (!b_mn) rc = make_tmap_2d_bf16(&maps.b[r], bp, K, N, ldb, DBK, bn);
    else rc = make_tmap_2d_bf16(&maps.b[r], bp, N, b_gather ? rows_b : K, ldb, 64, DBK);
    if (rc) return rc;
  }
  // staging applies to A sharded along M (K-major A) with more than one rank
  const bool stage_a = a_stage && chunk_flags && chunk_ctr && a_gather && !a_mn && W > 1 && (K % 8) == 0 &&
                       (lda % 8) == 0 && (ld_stage % 8) == 0;
  if (stage_a) {
    const int rc = make_tmap_2d_bf16(&maps.a_stage, a_stage, K, M, ld_stage, DBK, DBM);
    if (rc) return rc;
  } else {
    maps.a_stage = maps.a[rank];
  }
  DistParams p;
  p.a_stage = stage_a ? a_stage : nullptr; p.ld_stage = ld_stage; p.lda = lda;
  p.chunk_flags = stage_a ? chunk_flags : nullptr; p.chunk_ctr = stage_a ? chunk_ctr : nullptr;
  for (int r = 0; r < DMAXW; ++r) p.a_peer[r] = r < W ? a_ptrs[r] : nullptr;
  p.M = M; p.N = N; p.K = K; p.W = W; p.rank = rank;
  p.a_gather = a_gather; p.b_gather = b_gather; p.rows_a = rows_a; p.rows_b = rows_b;
  p.scatter = scatter;
  p.C = C; p.ldc = ldc; p.R = R; p.ldr = ldr;
  for (int r = 0; r < W; ++r) {
    p.stage[r] = stage_ptrs ? stage_ptrs[r] : nullptr;
    p.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  p.epoch = epoch;
  p.counters = counters;
  p.wait_ns = wait_ms > 0 ? static_cast<uint64_t>(wait_ms) * 1000000ull : 10000000000ull;
  p.status = status;
  const int tiles = ((M + DBM - 1) / DBM) * ((N + bn - 1) / bn);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  int rc;
#define SB_DISPATCH(BN_)                                                                     \
  do {                                                                                       \
    if (!a_mn && !b_mn) rc = launch_dist<BN_, false, false>(maps, p, grid, stream);          \
    else if (!a_mn && b_mn) rc = launch_dist<BN_, false, true>(maps, p, grid, stream);       \
    else if (a_mn && !b_mn) rc = launch_dist<BN_, true, false>(maps, p, grid, stream);       \
    else rc = launch_dist<BN_, true, true>(maps, p, grid, stream);                           \
  } while (0)
  if (bn == 256) SB_DISPATCH(256); else SB_DISPATCH(128);
#undef SB_DISPATCH
  return rc;
}
