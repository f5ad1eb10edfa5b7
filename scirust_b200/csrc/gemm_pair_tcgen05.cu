// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): one 256 x 256 output tile per pair of SMs.
//
// Same contract and operand forms as gemm_tcgen05.cu (C = op(A) * op(B), fp32 accumulation in tensor
// memory, optional bf16 residual, K walked in a fixed order). What changes is the traffic: the two
// CTAs of a cluster share one tcgen05.mma of M = 256, N = 256 per k-step. Each CTA stages its own
// 128 rows of A and only HALF of the B tile (128 of the 256 columns), so a CTA moves 32 KB per
// k-block for the same tensor work that costs 48 KB with 128 x 256 tiles per CTA, and six stages fit
// where four did. The accumulator rows of a CTA stay in its own TMEM; the epilogue is per CTA.
//
//   warp 0   TMA producer (both CTAs; bytes of both are counted on the leader's "full" barrier)
//   warp 1   MMA issuer (leader CTA only); the same warp allocates TMEM in both CTAs
//   warp 2-9 epilogue (both CTAs; "accumulator drained" arrives on the leader's barrier). The plain epilogue
//            (no SwiGLU, no split parts) does not store from registers: a warp converts 32 rows x 64 columns, lays
//            them out as 128-byte swizzled rows in its own 4 KB of shared memory and hands them to a TMA tensor
//            store, so the output leaves the SM as full 128-byte lines and edge tiles are clipped by the hardware
// Stage release and "accumulator ready" are tcgen05.commit arrivals delivered to both CTAs.
// No TMA multicast is used.
#include <cstdlib>
#include "sm100_ptx.cuh"
#include "api.h"
#include "gemm_sched.cuh"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int num_sms();

namespace pair {

constexpr int BM = 128;        // rows of A per CTA (256 per pair)
constexpr int BN = 256;        // columns of the pair's tile
constexpr int BNH = BN / 2;    // columns of B staged per CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 448;        // warp 0 TMA, 1 MMA, 2-9 epilogue, 10-13 all-gather copiers (idle otherwise)
constexpr int COPY_WARPS = 4;
constexpr int CP_UNROLL = 8;   // 16-byte peer loads in flight per copier thread
constexpr int GROUP_M = 8;           // row tiles (of 256 rows) per raster group
constexpr int MAXW = 8;
constexpr int FLAG_STRIDE = 16;     // flag words per phase in a call site's slot (as in gemm_dist_tcgen05.cu)
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB per CTA
constexpr int STAGES = 6;
constexpr int TMEM_COLS = 2 * BN;                // two accumulators
constexpr int EPI_WARPS = 8;
constexpr int EPI_STAGE_BYTES = 32 * 128;        // one warp's 32 rows x 64 bf16 columns, 128-byte swizzled rows
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * EPI_STAGE_BYTES + 1024 + 256;

struct TmapSet {
  CUtensorMap m[MAXW];   // reduce-scatter: the slot of this rank in every owner's receive buffer
};

struct Params {
  int M, N, K;
  void* C; int ldc;
  const void* R; int ldr;
  int* status;
  int use_tma_store;     // plain tiles leave through shared memory + TMA tensor store (tmap_c is valid)
  BalancedSched sched;   // workers are CTA pairs; see gemm_sched.cuh
  float* partials;       // dense fp32 [256, 256] blocks, one per scratch slot
  // SwiGLU epilogue (ff > 0): B is a fused [gate | up] weight of 2*ff columns and N == 2*ff. A tile then
  // holds 128 gate columns (staged by the leader CTA) and the MATCHING 128 up columns (staged by the
  // peer), so that after writing both to C the epilogue can also write act = silu(gate) * up.
  int ff;
  void* act; int ld_act;
  // SwiGLU-backward epilogue (gu != nullptr, ff == 0): the product is dh [M, N] (N = ff columns); instead
  // of storing it, the epilogue reads the saved [gate | up] row of the forward pass and writes
  // dgu = [dh * up * silu'(gate) | dh * silu(gate)] into C [M, 2N].
  const void* gu; int ld_gu;
  // All-gather -> GEMM (ag.W >= 1): A's rows are sharded over the ranks (rank s holds rows
  // [s*rows, (s+1)*rows) in its own buffer a_peer[s], row pitch lda). Every rank PUSHES its shard into the
  // landing buffers of all peers (stage_peer[r], peer-mapped, [M, ld_stage]; plain 16-byte stores, which, unlike
  // loads, need no round trip over NVLink): the copier warps of all CTAs share the copy for one destination at
  // a time, first the peer that needs this shard first (rank-1), then rank-2, ...; the warp that completes a
  // destination raises chunk_flags[source rank] there (one flag per source). The own shard is read in
  // place (tmap_a_own). The TMA producer waits (bounded) for the flag of the chunk it is about to read and walks
  // the row tiles in the matching rotated order (own rows, then rank+1's, ...). flags[r]: this call site's slot on
  // rank r; [1*16+s] "rank s has consumed its landing buffer": nobody leaves the kernel before every rank has,
  // so the next call's pushes cannot overwrite rows that a slower rank is still reading.
  struct {
    int W, rank, rows;
    const void* a_peer[MAXW]; int lda;     // only a_peer[rank] (the local shard) is read
    void* a_stage; int ld_stage;           // the local landing buffer (= stage_peer[rank])
    void* stage_peer[MAXW];
    int copy_own;                          // also place the own shard in the local landing buffer (nobody waits for
                                           // it: the caller wants the whole gathered matrix afterwards)
    uint32_t* flags[MAXW];
    uint32_t* chunk_flags;                 // local: chunk_flags[source rank], raised by the rank that pushed its shard
    uint32_t* chunk_flags_peer[MAXW];
    unsigned int* chunk_ctr; unsigned int* cta_ctr;
    uint32_t epoch;
    uint64_t wait_ns;
    int team;        // CTAs that share one chunk; teams work on different chunks at the same time
  } ag;
  // GEMM -> reduce-scatter (rs.W >= 1): every rank computes the partial product of ALL rows; rows
  // [o*rows, (o+1)*rows) belong to rank o. The epilogue PUSHES each finished tile straight into the owner's
  // receive buffer (p_peer[o] = rank o's buffer, bf16 [W sources][rows][ldc]; slot [my rank]) with a TMA tensor
  // store through the owner's tensor map, so the transfer over NVLink runs under the main loop of the following
  // tiles and nothing is left to pull at the end. Finished tiles are counted per 256-row block; when a block is
  // complete (its stores have been waited for) the rank raises "rank s's partial of this block has landed" on
  // the owner (ready[o] + s * blocks + block). The copier warps of the owner add the W slots of a block in rank
  // order 0..W-1 (+ residual) from LOCAL memory and write out [rows, ld_out]. Blocks of other owners are computed
  // first, own rows last, so the peers' pushes of my rows arrive while I compute theirs.
  struct {
    int W, rank, rows;
    const void* p_peer[MAXW];
    uint32_t* ready[MAXW];          // per rank: [W sources][rows / 256 blocks] epochs
    uint32_t* flags[MAXW];          // call-site slot: [1*16+s] "rank s has stopped reading my partial"
    unsigned int* block_ctr;        // [M / 256], zero on entry, reset by the kernel
    unsigned int* cta_ctr;
    void* out; int ld_out;
    const void* res; int ld_res;
    uint32_t epoch;
    uint64_t wait_ns;
    int team;        // CTAs that share one row block; teams reduce different blocks at the same time
  } rs;
};

__device__ __forceinline__ void p_st_release_sys(uint32_t* ptr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ void p_st_release_gpu(uint32_t* ptr, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
template <bool SYS>
__device__ bool p_wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns, int* status) {
  auto ld = [&]() {
    uint32_t v;
    if (SYS) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    else asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    return v;
  };
  if (static_cast<int32_t>(ld() - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld() - epoch) < 0) {
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

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_a_own, const __grid_constant__ CUtensorMap tmap_c,
                 const __grid_constant__ TmapSet tmap_rs, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES;      // EPI_WARPS x 4 KB, 1024-byte aligned
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + EPI_WARPS * EPI_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader, 1 = peer
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  const int mt2 = (p.M + 2 * BM - 1) / (2 * BM);
  const int nt = p.ff ? (p.ff + BNH - 1) / BNH : (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_total = mt2 * nt;
  // Tile order: groups of GROUP_M row tiles sweep all column tiles before the next group starts, so a
  // wave of CTA pairs touches few distinct A and B tiles (an A larger than L2 is then read from DRAM
  // once per group instead of once per column tile). The balanced schedule keeps plain n-major order,
  // which is what its fix-up pass assumes.
  const int group_m = p.sched.sk_tiles > 0 ? mt2 : (mt2 < GROUP_M ? mt2 : GROUP_M);
  auto tile_mn = [&](int t, int& m2, int& n_idx) {
    const int gsz = group_m * nt;
    const int g = t / gsz;
    const int first = g * group_m;
    const int gm = min(group_m, mt2 - first);
    const int within = t - g * gsz;
    n_idx = within / gm;
    m2 = first + (within - n_idx * gm);
  };
  const bool ag = p.ag.W >= 1;   // a one-rank group runs the same protocol with itself as the only peer
  const bool rs = p.rs.W >= 1;
  const int m_rot = ag ? p.ag.rank * (mt2 / p.ag.W)        // walk the local shard's row tiles first
                       : (rs ? ((p.rs.rank + 1) % p.rs.W) * (mt2 / p.rs.W) : 0);   // the next rank's rows first, own rows last

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);     // leader's producer arms it; both CTAs' copies complete on it
      mbar_init(&empty_bar[s], 1);    // one commit arrival (delivered to both CTAs)
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 16);  // 8 epilogue warps of each CTA arrive on the leader's barrier
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      SegIter iter(p.sched, pair_id, n_pairs, tiles_total, num_kb, 1, num_kb);
      Seg sg;
      while (ok && iter.next(sg)) {
        int n_idx, m2;
        tile_mn(sg.tile, m2, n_idx);
        m2 = (m2 + m_rot) % mt2;
        const int row0 = (m2 * 2 + static_cast<int>(rank)) * BM;      // this CTA's rows of A
        const int col0 = p.ff ? n_idx * BNH + static_cast<int>(rank) * p.ff   // gate half | matching up half
                              : n_idx * BN + static_cast<int>(rank) * BNH;   // this CTA's columns of B
        const bool own_rows = ag && row0 / p.ag.rows == p.ag.rank;   // read straight from the local shard
        const int row_own = row0 - (ag ? p.ag.rank * p.ag.rows : 0);
        if (ag && !own_rows && row0 < p.M) {
          // the shard of the rank that owns these rows must have landed in the local buffer
          if (!p_wait_flag<true>(p.ag.chunk_flags + row0 / p.ag.rows, p.ag.epoch, p.ag.wait_ns, p.status)) { ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy stores -> TMA reads
        }
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb_ = sa + A_BYTES;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if constexpr (!A_MN) {
            if (own_rows) tma_load_2d_pair(sa, &tmap_a_own, bar, kb * BK, row_own);
            else tma_load_2d_pair(sa, &tmap_a, bar, kb * BK, row0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d_pair(sa + c * (64 * BK * 2), &tmap_a, bar, row0 + c * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb_, &tmap_b, bar, kb * BK, col0);
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c)
              tma_load_2d_pair(sb_ + c * (64 * BK * 2), &tmap_b, bar, col0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      SegIter iter(p.sched, pair_id, n_pairs, tiles_total, num_kb, 1, num_kb);
      Seg sg;
      for (; ok && iter.next(sg); ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sb_ = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb_ + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc(sb_ + k * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage], 3);   // frees the stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 3);
      }
    }
  } else if (warp >= 10) {
    // -------------------------------- copiers (both CTAs) ---------------------------------
    if (ag && !A_MN && (p.ag.W > 1 || p.ag.copy_own)) {
      // Push my shard to every peer, one destination after the other (rank-1 first: it needs my rows first), all
      // CTAs sharing each destination's copy. One system fence per warp and destination; the warp that completes a
      // destination raises "rank's shard has landed" (chunk_flags[my rank]) there. Last, without any flag, the own
      // shard goes to the local landing buffer if the caller wants the whole gathered matrix.
      const int cw = warp - 10;
      const size_t vec_per_row = static_cast<size_t>(p.K) / 8;               // 16-byte words per row
      const size_t vecs = vec_per_row * p.ag.rows;                            // words of one shard
      const size_t lo = vecs * blockIdx.x / gridDim.x, hi = vecs * (blockIdx.x + 1) / gridDim.x;
      const uint4* mine = static_cast<const uint4*>(p.ag.a_peer[p.ag.rank]);
      const size_t srow0 = static_cast<size_t>(p.ag.rank) * p.ag.rows;       // my rows in the gathered matrix
      const int n_dst = p.ag.W - 1 + (p.ag.copy_own ? 1 : 0);
      // A shard of a few MB is pushed to all destinations before the one fence (the fence waits for the stores to be
      // acknowledged over NVLink, several microseconds each time, more than such a shard's GEMM gains by starting early);
      // larger shards fence and announce destination by destination, so the consumer starts on the first while the
      // others are still in flight.
      const bool announce_each = vecs * 16 > (static_cast<size_t>(8) << 20);
      for (int q = 1; q <= n_dst; ++q) {
        const int dst = (p.ag.rank + p.ag.W - q) % p.ag.W;                    // q == W: myself
        uint4* land = static_cast<uint4*>(p.ag.stage_peer[dst]);
        for (size_t v0 = lo + (cw * 32 + lane); v0 < hi; v0 += COPY_WARPS * 32 * CP_UNROLL) {
          uint4 tmp[CP_UNROLL];
          size_t idx[CP_UNROLL];
#pragma unroll
          for (int u = 0; u < CP_UNROLL; ++u) {
            idx[u] = v0 + static_cast<size_t>(u) * COPY_WARPS * 32;
            if (idx[u] < hi) {
              const size_t r = idx[u] / vec_per_row, c = idx[u] - r * vec_per_row;
              tmp[u] = __ldg(mine + (r * p.ag.lda) / 8 + c);
            }
          }
#pragma unroll
          for (int u = 0; u < CP_UNROLL; ++u) {
            if (idx[u] < hi) {
              const size_t r = idx[u] / vec_per_row, c = idx[u] - r * vec_per_row;
              *(land + ((srow0 + r) * p.ag.ld_stage) / 8 + c) = tmp[u];
            }
          }
        }
        if (dst == p.ag.rank || !announce_each) continue;
        __threadfence_system();        // this warp's stores have reached the destination
        __syncwarp();
        if (lane == 0) {
          const unsigned int prev = atomicAdd(p.ag.chunk_ctr + dst, 1u);
          if (prev + 1 == gridDim.x * COPY_WARPS) {
            __threadfence_system();
            p_st_release_sys(p.ag.chunk_flags_peer[dst] + p.ag.rank, p.ag.epoch);
          }
        }
      }
      if (!announce_each && p.ag.W > 1) {
        __threadfence_system();        // this warp's stores have reached every destination
        __syncwarp();
        if (lane == 0) {
          const unsigned int prev = atomicAdd(p.ag.chunk_ctr, 1u);
          if (prev + 1 == gridDim.x * COPY_WARPS) {
            __threadfence_system();
            for (int q = 1; q < p.ag.W; ++q)
              p_st_release_sys(p.ag.chunk_flags_peer[(p.ag.rank + p.ag.W - q) % p.ag.W] + p.ag.rank, p.ag.epoch);
          }
        }
      }
    }
    if (rs) {
      // ---- reduce-scatter: pull and add the partials of my row blocks as they complete ----
      const int cw = warp - 10;
      const int bpr = p.rs.rows / (2 * BM);                                   // my 256-row blocks
      const size_t vec_per_row = static_cast<size_t>(p.N) / 8;
      const size_t vec_per_block = vec_per_row * 2 * BM;
      const int team = p.rs.team, n_teams = gridDim.x / team;
      const int my_team = blockIdx.x / team, member = blockIdx.x - my_team * team;
      const size_t lo = vec_per_block * member / team, hi = vec_per_block * (member + 1) / team;
      const uint32_t* my_ready = p.rs.ready[p.rs.rank];
      for (int bi = my_team; bi < bpr && my_team < n_teams; bi += n_teams) {
        int okf = 1;
        if (lane == 0) {
          for (int sidx = 0; sidx < p.rs.W && okf; ++sidx)
            okf = p_wait_flag<true>(my_ready + sidx * bpr + bi, p.rs.epoch, p.rs.wait_ns, p.status) ? 1 : 0;
        }
        okf = __shfl_sync(0xffffffffu, okf, 0);
        if (!okf) break;
        const size_t lrow0 = static_cast<size_t>(bi) * 2 * BM;                      // first row of the block in my shard
        for (size_t v0 = lo + (cw * 32 + lane); v0 < hi; v0 += COPY_WARPS * 32 * 4) {
          // four 16-byte columns per thread and two sources at a time in flight; the sum runs in rank order
          float acc8[4][8];
          size_t off_p[4], off_l[4];
          bool live[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const size_t v = v0 + static_cast<size_t>(u) * COPY_WARPS * 32;
            live[u] = v < hi;
            const size_t r = live[u] ? v / vec_per_row : 0, c = live[u] ? (v - r * vec_per_row) * 8 : 0;
            off_p[u] = (lrow0 + r) * p.ldc + c;      // inside one source's slot of my receive buffer
            off_l[u] = (r << 20) | c;          // packed (row inside the block, column): N < 2^20
#pragma unroll
            for (int j = 0; j < 8; ++j) acc8[u][j] = 0.f;
          }
          for (int s0 = 0; s0 < p.rs.W; s0 += 2) {
            uint4 x[2][4];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (s0 + t < p.rs.W) {
                const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(p.rs.p_peer[p.rs.rank]) +
                                            static_cast<size_t>(s0 + t) * p.rs.rows * p.ldc;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  if (live[u])
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(x[t][u].x), "=r"(x[t][u].y), "=r"(x[t][u].z), "=r"(x[t][u].w)
                                 : "l"(base + off_p[u]) : "memory");
                }
              }
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              if (s0 + t < p.rs.W) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  if (live[u]) {
                    const uint4 y = x[t][u];
                    acc8[u][0] += bf16_lo(y.x); acc8[u][1] += bf16_hi(y.x); acc8[u][2] += bf16_lo(y.y); acc8[u][3] += bf16_hi(y.y);
                    acc8[u][4] += bf16_lo(y.z); acc8[u][5] += bf16_hi(y.z); acc8[u][6] += bf16_lo(y.w); acc8[u][7] += bf16_hi(y.w);
                  }
                }
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (!live[u]) continue;
            const size_t r = off_l[u] >> 20, c = off_l[u] & 0xfffff;
            if (p.rs.res) {
              const uint4 y = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.rs.res) +
                                                              (lrow0 + r) * p.rs.ld_res + c);
              acc8[u][0] += bf16_lo(y.x); acc8[u][1] += bf16_hi(y.x); acc8[u][2] += bf16_lo(y.y); acc8[u][3] += bf16_hi(y.y);
              acc8[u][4] += bf16_lo(y.z); acc8[u][5] += bf16_hi(y.z); acc8[u][6] += bf16_lo(y.w); acc8[u][7] += bf16_hi(y.w);
            }
            uint4 o;
            o.x = pack_bf16x2(acc8[u][0], acc8[u][1]); o.y = pack_bf16x2(acc8[u][2], acc8[u][3]);
            o.z = pack_bf16x2(acc8[u][4], acc8[u][5]); o.w = pack_bf16x2(acc8[u][6], acc8[u][7]);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.rs.out) + (lrow0 + r) * p.rs.ld_out + c) = o;
          }
        }
      }
    }
  } else {
    // -------------------------------- epilogue (both CTAs) --------------------------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t leader_empty0 = mapa_shared(smem_u32(&tmem_empty[0]), 0);
    const uint32_t leader_empty1 = mapa_shared(smem_u32(&tmem_empty[1]), 0);
    bool ok = true;
    int it = 0;
    // reduce-scatter: the row block whose stores (TMA, to the owner's memory) this CTA has issued but not yet
    // announced. A CTA's share of a tile counts once the stores of its eight epilogue warps are complete (each warp
    // waits for its own, then the warps meet at a named barrier and ONE thread pays for the system fence); the CTA
    // that completes a 256-row block raises the block's flag on its owner.
    int pend_m2 = -1;
    auto rs_announce = [&](int mb) {
      asm volatile("fence.proxy.async;" ::: "memory");     // the stores went through the async proxy
      __threadfence_system();
      const unsigned int prev = atomicAdd(p.rs.block_ctr + mb, 1u);
      if (prev + 1 == static_cast<unsigned int>(nt) * 2u) {
        const int bpr = p.rs.rows / (2 * BM);
        const int owner = mb / bpr;
        __threadfence_system();
        p_st_release_sys(p.rs.ready[owner] + p.rs.rank * bpr + (mb - owner * bpr), p.rs.epoch);
      }
    };
    SegIter iter(p.sched, pair_id, n_pairs, tiles_total, num_kb, 1, num_kb);
    Seg sg;
    for (; ok && iter.next(sg); ++it) {
      int n_idx, m2;
      tile_mn(sg.tile, m2, n_idx);
      m2 = (m2 + m_rot) % mt2;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = (m2 * 2 + static_cast<int>(rank)) * BM + q * 32 + lane;
      const uint32_t taddr_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (p.ff) {
        // SwiGLU tile: accumulator columns [0,128) are gate, [128,256) the matching up columns
#pragma unroll 1
        for (int gc = half * 2; gc < half * 2 + 2; ++gc) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr_row + gc * 32, rg);
          tmem_ld_32x32(taddr_row + BNH + gc * 32, ru);
          tmem_ld_wait();
          const int gcol = n_idx * BNH + gc * 32;
          if (row < p.M && gcol < p.ff) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc;
            __nv_bfloat16* arow = reinterpret_cast<__nv_bfloat16*>(p.act) + static_cast<size_t>(row) * p.ld_act;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (gcol + v * 8 < p.ff) {   // ff % 8 == 0 is enforced on the host
                uint4 og, ou, oa;
                uint32_t* pg = &og.x; uint32_t* pu = &ou.x; uint32_t* pa = &oa.x;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  pg[j] = pack_bf16x2(__uint_as_float(rg[v * 8 + 2 * j]), __uint_as_float(rg[v * 8 + 2 * j + 1]));
                  pu[j] = pack_bf16x2(__uint_as_float(ru[v * 8 + 2 * j]), __uint_as_float(ru[v * 8 + 2 * j + 1]));
                  // act from the bf16-rounded gate / up, exactly what the stand-alone kernel reads back
                  const float g0 = bf16_lo(pg[j]), g1 = bf16_hi(pg[j]);
                  const float u0 = bf16_lo(pu[j]), u1 = bf16_hi(pu[j]);
                  pa[j] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                }
                *reinterpret_cast<uint4*>(crow + gcol + v * 8) = og;
                *reinterpret_cast<uint4*>(crow + p.ff + gcol + v * 8) = ou;
                *reinterpret_cast<uint4*>(arow + gcol + v * 8) = oa;
              }
            }
          }
        }
      } else if (!p.gu && sg.slot < 0 && p.use_tma_store) {
        // plain tile through shared memory and a TMA tensor store: two slabs of 64 columns per warp
        uint8_t* stg = epi_stage + (warp - 2) * EPI_STAGE_BYTES;
        const int row0w = (m2 * 2 + static_cast<int>(rank)) * BM + q * 32;      // first row of this warp
#pragma unroll 1
        for (int sl = 0; sl < 2; ++sl) {
          const int colw = n_idx * BN + half * (BN / 2) + sl * 64;
          if (lane == 0) tma_store_wait_read<0>();      // the previous slab has left the staging buffer
          __syncwarp();
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t r[32];
            tmem_ld_32x32(taddr_row + (half * (BN / 64) + sl * 2 + cc) * 32, r);
            tmem_ld_wait();
            const int col0 = colw + cc * 32;
            const __nv_bfloat16* rrow = (p.R && row < p.M && col0 < p.N)
                ? reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr + col0 : nullptr;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              if (rrow && col0 + v * 8 < p.N) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + v * 8);
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
              const int chunk = cc * 4 + v;              // 16-byte chunk of the 128-byte row
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = o;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          const bool issued = row0w < p.M && colw < p.N;    // a slab wholly past the edge stores nothing
          if (lane == 0 && issued) {
            if (rs) {
              const int owner = m2 / (p.rs.rows / (2 * BM));
              tma_store_2d(&tmap_rs.m[owner], stg, colw, row0w - owner * p.rs.rows);
            } else {
              tma_store_2d(&tmap_c, stg, colw, row0w);
            }
            tma_store_commit();
          }
          if (rs && sl == 0 && pend_m2 >= 0) {
            // all but the group just committed are complete: the previous tile has landed on its owner
            if (lane == 0) {
              if (issued) tma_store_wait<1>(); else tma_store_wait<0>();
              asm volatile("fence.proxy.async;" ::: "memory");
            }
            __syncwarp();
            asm volatile("bar.sync 2, 256;" ::: "memory");      // the eight epilogue warps of this CTA
            if (warp == 2 && lane == 0) rs_announce(pend_m2);
            pend_m2 = -1;
          }
        }
      } else {
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c * 32, r);
        tmem_ld_wait();
        if (p.gu) {
          const int col = n_idx * BN + c * 32;
          if (row < p.M && col < p.N) {
            const __nv_bfloat16* grow = reinterpret_cast<const __nv_bfloat16*>(p.gu) + static_cast<size_t>(row) * p.ld_gu;
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col + v * 8 < p.N) {
                const uint4 gv = *reinterpret_cast<const uint4*>(grow + col + v * 8);
                const uint4 uv = *reinterpret_cast<const uint4*>(grow + p.N + col + v * 8);
                const uint32_t* pg = &gv.x; const uint32_t* pu = &uv.x;
                uint4 odg, odu;
                uint32_t* qg = &odg.x; uint32_t* qu = &odu.x;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  // dh rounded to bf16 first: the stand-alone kernel reads it back from a bf16 tensor
                  const uint32_t dpk = pack_bf16x2(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                  const float d0 = bf16_lo(dpk), d1 = bf16_hi(dpk);
                  const float g0 = bf16_lo(pg[j]), g1 = bf16_hi(pg[j]);
                  const float u0 = bf16_lo(pu[j]), u1 = bf16_hi(pu[j]);
                  const float s0 = 1.f / (1.f + __expf(-g0)), s1 = 1.f / (1.f + __expf(-g1));
                  qg[j] = pack_bf16x2(d0 * u0 * s0 * (1.f + g0 * (1.f - s0)), d1 * u1 * s1 * (1.f + g1 * (1.f - s1)));
                  qu[j] = pack_bf16x2(d0 * g0 * s0, d1 * g1 * s1);
                }
                *reinterpret_cast<uint4*>(crow + col + v * 8) = odg;
                *reinterpret_cast<uint4*>(crow + p.N + col + v * 8) = odu;
              }
            }
          }
          continue;
        }
        const int col0 = n_idx * BN + c * 32;
        if (sg.slot >= 0) {
          // part of a tile of the balanced schedule: this CTA's 128 rows of the pair's fp32 block
          float* prow = p.partials +
                        (static_cast<size_t>(sg.slot) * (2 * BM) + rank * BM + (q * 32 + lane)) * BN + c * 32;
#pragma unroll
          for (int v = 0; v < 8; ++v)
            *reinterpret_cast<uint4*>(prow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        } else if (row < p.M && col0 < p.N) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
          const __nv_bfloat16* rrow =
              p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr + col0 : nullptr;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p.N) {  // N % 8 == 0 is enforced on the host
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              if (rrow) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + v * 8);
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
              *reinterpret_cast<uint4*>(crow + v * 8) = o;
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
      if (rs) pend_m2 = m2;     // announced once its stores have completed (during the next tile, or below)
    }
    if (rs && pend_m2 >= 0) {
      if (lane == 0) {
        tma_store_wait<0>();
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      __syncwarp();
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (warp == 2 && lane == 0) rs_announce(pend_m2);
    }
  }

  if (warp >= 2 && warp < 2 + EPI_WARPS && lane == 0) tma_store_wait<0>();   // staged output has left shared memory
  // Teardown: every role loop is bounded, so all threads of both CTAs arrive here. Neither CTA may
  // leave while the other can still read its shared memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
  if (rs && threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(p.rs.cta_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *p.rs.cta_ctr = 0;
      for (int i = 0; i < mt2; ++i) p.rs.block_ctr[i] = 0;
      if (*reinterpret_cast<volatile int*>(p.status) == 0) {
        // every CTA of this rank has finished pulling: the peers may overwrite their partials; stay until
        // the peers have finished pulling mine
        __threadfence_system();
        for (int r = 0; r < p.rs.W; ++r) p_st_release_sys(p.rs.flags[r] + 1 * FLAG_STRIDE + p.rs.rank, p.rs.epoch);
        for (int sidx = 0; sidx < p.rs.W; ++sidx)
          if (!p_wait_flag<true>(p.rs.flags[p.rs.rank] + 1 * FLAG_STRIDE + sidx, p.rs.epoch, p.rs.wait_ns, p.status)) break;
      }
    }
  }
  if (ag && threadIdx.x == 0) {
    // last CTA: reset the counters; tell the peers this rank has consumed its landing buffer and stay until every
    // peer has consumed its own (all pushes of this call have then been read, and the next call may push again)
    __threadfence();
    const unsigned int prev = atomicAdd(p.ag.cta_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *p.ag.cta_ctr = 0;
      for (int i = 0; i < p.ag.W; ++i) p.ag.chunk_ctr[i] = 0;      // one counter per destination
      if (*reinterpret_cast<volatile int*>(p.status) == 0) {
        __threadfence_system();
        for (int r = 0; r < p.ag.W; ++r) p_st_release_sys(p.ag.flags[r] + 1 * FLAG_STRIDE + p.ag.rank, p.ag.epoch);
        for (int s = 0; s < p.ag.W; ++s)
          if (!p_wait_flag<true>(p.ag.flags[p.ag.rank] + 1 * FLAG_STRIDE + s, p.ag.epoch, p.ag.wait_ns, p.status)) break;
      }
    }
  }
}

// Number of CTA pairs the device keeps resident at once (the kernel runs one CTA per SM).
static int max_pairs() {
  static int cached = 0;
  if (!cached) {
    auto kern = gemm_pair_kernel<false, false>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * (num_sms() / 2));
    q.blockDim = dim3(THREADS);
    q.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
    q.attrs = qa; q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n < 1) n = num_sms() / 2;
    if (n > num_sms() / 2) n = num_sms() / 2;
    cached = n;
  }
  return cached;
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int grid, cudaStream_t stream,
                  const CUtensorMap* ta_own = nullptr, const CUtensorMap* tc = nullptr, const TmapSet* trs = nullptr) {
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  static const TmapSet none = {};
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, ta_own ? *ta_own : ta, tc ? *tc : ta, trs ? *trs : none, p) ==
                 cudaSuccess
             ? 0
             : SB_ERR_LAUNCH;
}

}  // namespace pair
}  // namespace sb

using namespace sb;

// Same contract as sb_gemm_bf16 without split-K: C[M,N] (bf16) = op(A) op(B) (+ R). M, N, K > 0,
// N % 8 == 0, leading dimensions multiples of 8 elements, 16-byte aligned bases.
// `workspace` (optional): sb_gemm_pair_workspace_floats() floats; with it the balanced schedule is used.
// `gu` (optional, with ff == 0): SwiGLU-backward epilogue. The product is dh [M, N]; C must be [M, 2N] and
// receives dgu computed from the saved forward [gate | up] rows `gu` [M, ld_gu]; no residual.
// `act` (optional, with ff > 0): SwiGLU epilogue. B then holds [gate | up] (N == 2*ff, ff % 8 == 0), C receives
// the bf16 [gate | up] product as usual and `act` [M, ld_act] receives silu(gate) * up; no residual, no
// balanced schedule on that path.
extern "C" size_t sb_gemm_pair_workspace_floats() { return static_cast<size_t>(num_sms() / 2) * 3 * 256 * 256; }

extern "C" int sb_gemm_pair_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda,
                                 int ldb, int ldc, int ldr, int a_mn, int b_mn, void* workspace, void* act, int ld_act,
                                 int ff, const void* gu, int ld_gu, int* status, void* stream_) {
  using namespace sb::pair;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (ldc & 7) || (R && (ldr & 7))) return SB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (R && (reinterpret_cast<uintptr_t>(R) & 15))) return SB_ERR_ALIGN;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  else rc = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BNH);
  else rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  if (ff) {
    if (!act || N != 2 * ff || (ff & 7) || (ld_act & 7) || R || (reinterpret_cast<uintptr_t>(act) & 15)) return SB_ERR_ARG;
    workspace = nullptr;
  }
  Params p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.R = R; p.ldr = ldr; p.status = status;
  p.ff = ff; p.act = act; p.ld_act = ld_act;
  if (gu) {
    if (ff || R || (ld_gu & 7) || (reinterpret_cast<uintptr_t>(gu) & 15)) return SB_ERR_ARG;
    workspace = nullptr;
  }
  p.gu = gu; p.ld_gu = ld_gu;
  p.ag.W = 0;
  p.rs.W = 0;
  // output through shared memory + TMA tensor store (SB_GEMM_TMA_STORE=0 keeps the register stores)
  static const bool tma_store = [] { const char* e = getenv("SB_GEMM_TMA_STORE"); return !(e && e[0] == '0'); }();
  CUtensorMap tc;
  p.use_tma_store = 0;
  if (tma_store && !ff && !gu) {
    rc = make_tmap_2d_bf16(&tc, C, N, M, ldc, 64, 32);
    if (rc) return rc;
    p.use_tma_store = 1;
  }
  const int mt2 = (M + 2 * BM - 1) / (2 * BM), nt = ff ? (ff + BNH - 1) / BNH : (N + BN - 1) / BN;
  const int num_kb = (K + BK - 1) / BK;
  const int pairs_avail = max_pairs();
  const int tiles = mt2 * nt;
  int pairs = tiles < pairs_avail ? tiles : pairs_avail;
  bool fixup = false;
  p.partials = nullptr;
  if (workspace && plan_balanced(tiles, num_kb, pairs_avail, &p.sched, &fixup)) {
    p.partials = static_cast<float*>(workspace);
    pairs = p.sched.dp_tiles > 0 ? pairs_avail : p.sched.sk_workers;
  } else {
    p.sched.dp_tiles = p.sched.sk_tiles = p.sched.sk_workers = p.sched.sk_slots = 0;
  }
  const int grid = 2 * pairs;
  const CUtensorMap* tcp = p.use_tma_store ? &tc : nullptr;
  if (!a_mn && !b_mn) rc = launch<false, false>(ta, tb, p, grid, stream, nullptr, tcp);
  else if (!a_mn && b_mn) rc = launch<false, true>(ta, tb, p, grid, stream, nullptr, tcp);
  else if (a_mn && !b_mn) rc = launch<true, false>(ta, tb, p, grid, stream, nullptr, tcp);
  else rc = launch<true, true>(ta, tb, p, grid, stream, nullptr, tcp);
  if (rc) return rc;
  if (fixup) {
    dim3 fg(p.sched.sk_tiles, 2 * BM * BN / (256 * 4));
    balanced_fixup_kernel<2 * BM, BN><<<fg, 256, 0, stream>>>(p.sched, p.partials, static_cast<__nv_bfloat16*>(C), ldc,
                                                             static_cast<const __nv_bfloat16*>(R), ldr, M, N, mt2,
                                                             num_kb);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  return 0;
}

// All-gather -> GEMM on CTA pairs: C[M,N] = gather(A shards)[M,K] * op(B) (+ R). a_ptrs[s]: rank s's shard
// [M/W, lda] (only entry `rank`, the local one, is read); stage_ptrs[r]: rank r's landing buffer [M, ld_stage]
// (peer-mapped: every rank pushes its shard into every peer's); flag_ptrs[r]: this call site's flag slot on rank r;
// chunk_flag_ptrs[r]: rank r's per-source epochs (peer-mapped, >= W words, zero when created); chunk_ctr: >= W local words,
// cta_ctr one local word (zero on entry, left zero). (M / W) % 256 == 0, K % 8 == 0. B is local ([K,N] when b_mn,
// else [N,K]). copy_own != 0: the own shard is copied into the local landing buffer too, which then holds the whole
// gathered matrix when the kernel has finished (weight-gradient products reuse it instead of gathering again).
extern "C" int sb_gemm_pair_ag_bf16(void* const* a_ptrs, const void* B, void* C, const void* R, int M, int N, int K,
                                    int lda, int ldb, int ldc, int ldr, int b_mn, void* const* stage_ptrs, int ld_stage,
                                    void* const* flag_ptrs, void* const* chunk_flag_ptrs, unsigned int* chunk_ctr,
                                    unsigned int* cta_ctr, int rank, int W, uint32_t epoch, int wait_ms, int copy_own,
                                    int* status, void* stream_) {
  using namespace sb::pair;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || W < 1 || W > MAXW || rank < 0 || rank >= W) return SB_ERR_ARG;
  if ((N & 7) || (K & 7) || (lda & 7) || (ld_stage & 7) || (ldc & 7) || (R && (ldr & 7)) || (M % (W * 2 * BM)))
    return SB_ERR_ARG;
  void* a_stage = stage_ptrs[rank];
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(a_stage) & 15)) return SB_ERR_ALIGN;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, a_stage, K, M, ld_stage, BK, BM);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BNH);
  else rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  Params p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.R = R; p.ldr = ldr; p.status = status;
  p.ff = 0; p.act = nullptr; p.ld_act = 0; p.gu = nullptr; p.ld_gu = 0;
  p.partials = nullptr;
  p.use_tma_store = 0;
  p.sched.dp_tiles = p.sched.sk_tiles = p.sched.sk_workers = p.sched.sk_slots = 0;
  p.rs.W = 0;
  p.ag.W = W; p.ag.rank = rank; p.ag.rows = M / W; p.ag.lda = lda;
  p.ag.a_stage = a_stage; p.ag.ld_stage = ld_stage;
  for (int r = 0; r < MAXW; ++r) {
    p.ag.a_peer[r] = r < W ? a_ptrs[r] : nullptr;
    p.ag.flags[r] = r < W ? static_cast<uint32_t*>(flag_ptrs[r]) : nullptr;
    p.ag.stage_peer[r] = r < W ? stage_ptrs[r] : nullptr;
    p.ag.chunk_flags_peer[r] = r < W ? static_cast<uint32_t*>(chunk_flag_ptrs[r]) : nullptr;
  }
  p.ag.chunk_flags = static_cast<uint32_t*>(chunk_flag_ptrs[rank]); p.ag.chunk_ctr = chunk_ctr; p.ag.cta_ctr = cta_ctr;
  p.ag.copy_own = copy_own;
  p.ag.epoch = epoch;
  p.ag.wait_ns = wait_ms > 0 ? static_cast<uint64_t>(wait_ms) * 1000000ull : 10000000000ull;
  // every CTA pair runs copier warps, so the whole device is launched whatever the tile count
  const int grid = 2 * max_pairs();
  CUtensorMap ta_own;
  rc = make_tmap_2d_bf16(&ta_own, a_ptrs[rank], K, M / W, lda, BK, BM);
  if (rc) return rc;
  // a team of CTAs shares one 128-row chunk so that every member moves about 32 KB of it
  const long long chunk_bytes = static_cast<long long>(BM) * K * 2;
  int team = static_cast<int>((chunk_bytes + 32767) / 32768);
  if (team < 1) team = 1;
  if (team > grid) team = grid;
  team = grid / (grid / team);      // as few idle CTAs as the grid allows
  p.ag.team = team;
  CUtensorMap tc;
  rc = make_tmap_2d_bf16(&tc, C, N, M, ldc, 64, 32);
  if (rc) return rc;
  p.use_tma_store = 1;
  if (!b_mn) return launch<false, false>(ta, tb, p, grid, stream, &ta_own, &tc);
  return launch<false, true>(ta, tb, p, grid, stream, &ta_own, &tc);
}

// GEMM -> reduce-scatter on CTA pairs: out[M/W, N] = rows of this rank of sum over ranks (A_r * op(B_r)) (+ res).
// part_ptrs[s]: rank s's partial buffer [M, ldp] (symmetric memory, peer-mapped; entry `rank` is the local
// one this call writes); ready_ptrs[r]: rank r's [W][M/W/256] epoch words; flag_ptrs[r]: the call site's flag
// slot on rank r; block_ctr: M/256 words, cta_ctr: one word (zero on entry, left zero). (M / W) % 256 == 0.
extern "C" int sb_gemm_pair_rs_bf16(const void* A, const void* B, void* const* part_ptrs, int ldp, void* out, int ld_out,
                                    const void* res, int ld_res, int M, int N, int K, int lda, int ldb, int b_mn,
                                    void* const* ready_ptrs, void* const* flag_ptrs, unsigned int* block_ctr,
                                    unsigned int* cta_ctr, int rank, int W, uint32_t epoch, int wait_ms, int* status,
                                    void* stream_) {
  using namespace sb::pair;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || W < 1 || W > MAXW || rank < 0 || rank >= W) return SB_ERR_ARG;
  if ((N & 7) || (ldp & 7) || (ld_out & 7) || (res && (ld_res & 7)) || (M % (W * 2 * BM))) return SB_ERR_ARG;
  void* C = part_ptrs[rank];     // this rank's receive buffer [W][M / W][ldp]: the reducer reads it locally
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return SB_ERR_ALIGN;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BNH);
  else rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  // slot [rank] of every owner's receive buffer: [M / W rows][N columns], row pitch ldp
  TmapSet trs = {};
  for (int o = 0; o < W; ++o) {
    const __nv_bfloat16* slot = static_cast<const __nv_bfloat16*>(part_ptrs[o]) + static_cast<size_t>(rank) * (M / W) * ldp;
    rc = make_tmap_2d_bf16(&trs.m[o], slot, N, M / W, ldp, 64, 32);
    if (rc) return rc;
  }
  Params p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldp; p.R = nullptr; p.ldr = 0; p.status = status;
  p.ff = 0; p.act = nullptr; p.ld_act = 0; p.gu = nullptr; p.ld_gu = 0;
  p.partials = nullptr;
  p.use_tma_store = 1;           // reduce-scatter tiles always leave by TMA store, into the owners' memory
  p.sched.dp_tiles = p.sched.sk_tiles = p.sched.sk_workers = p.sched.sk_slots = 0;
  p.ag.W = 0;
  p.rs.W = W; p.rs.rank = rank; p.rs.rows = M / W;
  for (int r = 0; r < MAXW; ++r) {
    p.rs.p_peer[r] = r < W ? part_ptrs[r] : nullptr;
    p.rs.ready[r] = r < W ? static_cast<uint32_t*>(ready_ptrs[r]) : nullptr;
    p.rs.flags[r] = r < W ? static_cast<uint32_t*>(flag_ptrs[r]) : nullptr;
  }
  p.rs.block_ctr = block_ctr; p.rs.cta_ctr = cta_ctr;
  p.rs.out = out; p.rs.ld_out = ld_out; p.rs.res = res; p.rs.ld_res = ld_res;
  p.rs.epoch = epoch;
  p.rs.wait_ns = wait_ms > 0 ? static_cast<uint64_t>(wait_ms) * 1000000ull : 10000000000ull;
  const int grid = 2 * max_pairs();
  const long long block_bytes = static_cast<long long>(2 * BM) * N * 2 * W;   // bytes read per 256-row block
  int team = static_cast<int>((block_bytes + 65535) / 65536);
  if (team < 1) team = 1;
  if (team > grid) team = grid;
  team = grid / (grid / team);      // as few idle CTAs as the grid allows
  p.rs.team = team;
  if (!b_mn) return launch<false, false>(ta, tb, p, grid, stream, nullptr, nullptr, &trs);
  return launch<false, true>(ta, tb, p, grid, stream, nullptr, nullptr, &trs);
}
