// GQA flash-attention backward for sm_100a on tcgen05 tensor cores, without atomics.
//
// Three launches:
//   1. delta[b,h,s] = sum_d dO * O                                   (bandwidth-bound)
//   2. dK/dV: one CTA per (128-row kv tile, kv head, batch); loops over the query heads of
//      the group and over query tiles in ascending order, accumulating dK and dV in tensor
//      memory:  S^T = K Q^T,  dP^T = V dO^T,  dV += P^T dO,  dK += dS^T Q
//   3. dQ: one CTA per (128-row query tile, head, batch); loops over kv tiles in ascending
//      order:   S = Q K^T,  dP = dO V^T,  dQ += dS K
// Every sum has a fixed order, so gradients are bitwise repeatable (the reference gets the
// same property from per-(sequence, head) serial launches: cuda_model.rs:948-999, and
// softmax_bwd / scale_mask_bwd in scirust-cuda/src/chain.rs:479,337).
//
// P is recomputed from the saved log-sum-exp; dS = P * (dP - delta) * scale.
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t box0, uint32_t box1);
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

constexpr int BT = 128;          // tile edge (query rows and kv rows)
constexpr int BWD_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 softmax (two per TMEM lane quarter)
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  int B, S, H, Hkv;
  int ld_dqkv;
  float scale, scale_log2;
  int causal;
  const float* lse;    // [B,H,S]
  const float2* stats; // [B,H,S] (lse * log2(e), delta), written by attn_delta_kernel
  __nv_bfloat16* dqkv; // [B*S, ld_dqkv]
  int* status;
  int spill_ds;        // dK/dV kernel also stores every dS tile to the [B*H, S, S] scratch (see dQ below)
};

// Store 32 bf16 (packed in 16 words) of row r, columns [c*32, c*32+32) into a [128 x 128] bf16 tile
// laid out as two 128-byte-swizzled K-major chunks of 64 columns.
__device__ __forceinline__ void store_row32_sw128(uint8_t* tile, int r, int c, const uint32_t* pk) {
  uint8_t* prow = tile + (c >> 1) * (BT * 128) + r * 128;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int unit = ((c & 1) * 4 + u) ^ (r & 7);
    *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Element-wise core of both backward kernels for 32 score columns of one query row (thread = query
// row r, TMEM lane r): p = 2^(s*sl2 - lse2), dS = p * (dP*scale - delta*scale); columns beyond
// `lim` are masked. Writes dS (and P when WRITE_P) as bf16 into the swizzled [q x kv] tiles.
template <bool MASK, bool WRITE_P>
__device__ __forceinline__ void bwd_chunk(uint32_t tm_S, uint32_t tm_dP, uint32_t lane_off, int c, int r, int lim,
                                          float sl2, float lse2, float delta_s, float scale, uint8_t* p_buf,
                                          uint8_t* ds_buf) {
  uint32_t sv[32], dv[32];
  tmem_ld_32x32(tm_S + lane_off + c * 32, sv);
  tmem_ld_32x32(tm_dP + lane_off + c * 32, dv);
  tmem_ld_wait();
  uint32_t pk[16], dk[16];
  const float neg_lse2 = -lse2, neg_delta = -delta_s;
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    // packed pairs: (s0, s1) * sl2 - lse2, (dP0, dP1) * scale - delta * scale, p * (...)
    fma2(sv[i], sv[i + 1], sl2, neg_lse2);
    fma2(dv[i], dv[i + 1], scale, neg_delta);
    float p0 = fast_exp2(__uint_as_float(sv[i]));
    float p1 = fast_exp2(__uint_as_float(sv[i + 1]));
    if (MASK) {
      if (c * 32 + i > lim) p0 = 0.f;
      if (c * 32 + i + 1 > lim) p1 = 0.f;
    }
    mul2(dv[i], dv[i + 1], p0, p1);
    if (WRITE_P) pk[i >> 1] = pack_bf16x2(p0, p1);
    dk[i >> 1] = pack_bf16x2(__uint_as_float(dv[i]), __uint_as_float(dv[i + 1]));
  }
  if (WRITE_P) store_row32_sw128(p_buf, r, c, pk);
  store_row32_sw128(ds_buf, r, c, dk);
}

// --------------------------------------------------------------------------- delta
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  const float* __restrict__ lse, float2* __restrict__ stats, int B, int S, int H,
                                  int dh, int ld_o, int ld_do) {
  // a group of dh/8 lanes (8 or 16) owns one (token, head): 16-byte loads, then a butterfly inside the group
  const int gl = dh >> 3;                       // lanes per group
  const int gpw = 32 / gl;                      // groups per warp
  const int lane = threadIdx.x & 31;
  const int sub = lane % gl;
  const long long w = (static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * gpw + lane / gl;
  const bool live = w < static_cast<long long>(B) * S * H;
  float acc = 0.f;
  int row = 0, h = 0;
  if (live) {
    row = static_cast<int>(w / H);
    h = static_cast<int>(w - static_cast<long long>(row) * H);
    const uint4 a = *reinterpret_cast<const uint4*>(o + static_cast<size_t>(row) * ld_o + h * dh + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + static_cast<size_t>(row) * ld_do + h * dh + sub * 8);
    acc = bf16_lo(a.x) * bf16_lo(g.x) + bf16_hi(a.x) * bf16_hi(g.x) + bf16_lo(a.y) * bf16_lo(g.y) +
          bf16_hi(a.y) * bf16_hi(g.y) + bf16_lo(a.z) * bf16_lo(g.z) + bf16_hi(a.z) * bf16_hi(g.z) +
          bf16_lo(a.w) * bf16_lo(g.w) + bf16_hi(a.w) * bf16_hi(g.w);
  }
  for (int o2 = gl >> 1; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (live && sub == 0) {
    const int b = row / S, s = row - b * S;
    const size_t idx = (static_cast<size_t>(b) * H + h) * S + s;
    stats[idx] = make_float2(lse[idx] * LOG2E, acc);
  }
}

// --------------------------------------------------------------------------- dK / dV
// Pipeline (DH == 64): the bf16 P^T / dS^T tiles are double-buffered in shared memory, so the MMA
// warp issues the score products of iteration t+1 *before* the gradient products of iteration t;
// the softmax warps then work on t+1 while the tensor cores finish t. With DH == 128 shared
// memory only fits single buffers and the two groups are issued in program order.
template <int DH>
struct DkvCfg {
  static constexpr bool PDB = (DH == 64);             // double-buffer P^T / dS^T
  static constexpr int NPB = PDB ? 2 : 1;
  static constexpr int QS = (DH == 64) ? 2 : 1;       // (Q, dO) ring stages
  static constexpr int T_BYTES = BT * DH * 2;         // one [128 x DH] tile
  static constexpr int PT_BYTES = BT * BT * 2;
  static constexpr int TILE_BYTES = 2 * T_BYTES + QS * 2 * T_BYTES + NPB * 2 * PT_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 1024 + 128;
  static constexpr int TMEM_COLS = 512;  // S^T 128 | dP^T 128 | dK DH | dV DH
};

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                         const __grid_constant__ CUtensorMap tm_ds, const BwdParams p) {
  using Cfg = DkvCfg<DH>;
  constexpr int NCH = DH / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::T_BYTES;
  uint8_t* sQ = sV + Cfg::T_BYTES;                 // QS stages
  uint8_t* sdO = sQ + Cfg::QS * Cfg::T_BYTES;      // QS stages
  uint8_t* sPT = sdO + Cfg::QS * Cfg::T_BYTES;     // NPB buffers
  uint8_t* sdST = sPT + Cfg::NPB * Cfg::PT_BYTES;  // NPB buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdST + Cfg::NPB * Cfg::PT_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;            // QS
  uint64_t* q_empty = q_full + Cfg::QS;   // QS
  uint64_t* st_full = q_empty + Cfg::QS;
  uint64_t* p_full = st_full + 1;
  uint64_t* done = p_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (p.S + BT - 1) / BT;
  // The kv tile is the slowest grid index: CTAs are handed out in block-id order, so all the long tiles
  // (causal: small kt, up to 4x16 query tiles) start first and the short ones fill the tail.
  const int kt = blockIdx.z;  // kv tile
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int group = p.H / p.Hkv;
  const int kv0 = kt * BT;
  const int row_base = b * p.S;
  const int qt_first = p.causal ? kt : 0;
  const int n_qt = n_t - qt_first;
  const int n_iter = group * n_qt;  // iteration t -> head kvh*group + t / n_qt, q tile qt_first + t % n_qt

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < Cfg::QS; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(st_full, 1);
    mbar_init(p_full, 8);  // one arrival per softmax warp
    mbar_init(done, 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tm_qkv); prefetch_tmap(&tm_do); }
  if (warp == 1) { tmem_alloc(tmem_holder, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  // S and dP are [query x kv] (TMEM lane = query row, as in the dQ kernel); their bf16 images P and dS
  // are stored [q rows][kv] and consumed as MN-major A operands (A^T) by the dV / dK products.
  const uint32_t tm_ST = tmem_base, tm_dPT = tmem_base + 128, tm_dK = tmem_base + 256, tm_dV = tmem_base + 256 + DH;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::T_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tma_load_2d(sK + c * (BT * 128), &tm_qkv, kv_full, (p.H + kvh) * DH + c * 64, row_base + kv0);
        tma_load_2d(sV + c * (BT * 128), &tm_qkv, kv_full, (p.H + p.Hkv + kvh) * DH + c * 64, row_base + kv0);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int t = 0; t < n_iter; ++t) {
        const int head = kvh * group + t / n_qt;
        const int qt = qt_first + t % n_qt;
        if (!mbar_wait(&q_empty[st], ph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&q_full[st], 2 * Cfg::T_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sQ + st * Cfg::T_BYTES + c * (BT * 128), &tm_qkv, &q_full[st], head * DH + c * 64,
                      row_base + qt * BT);
          tma_load_2d(sdO + st * Cfg::T_BYTES + c * (BT * 128), &tm_do, &q_full[st], head * DH + c * 64,
                      row_base + qt * BT);
        }
        if (++st == Cfg::QS) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BT, BT, false, false);   // [q x kv], both K-major
      constexpr uint32_t idesc_g = make_idesc_bf16(BT, DH, true, true);     // [kv x dh] = A^T B, both MN-major
      bool ok = mbar_wait(kv_full, 0, p.status, ST_TIMEOUT_FULL);
      int st_s = 0;          // stage / phase of the next score issue
      uint32_t ph_s = 0;
      int st_g = 0;          // stage of the next gradient issue
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      auto issue_scores = [&]() -> bool {
        if (!mbar_wait(&q_full[st_s], ph_s, p.status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t bQ = smem_u32(sQ + st_s * Cfg::T_BYTES), bdO = smem_u32(sdO + st_s * Cfg::T_BYTES);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = (k >> 2) * (BT * 128) + (k & 3) * 32;
          umma_bf16_ss(tm_ST, make_smem_desc(bQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024), idesc_s,
                       k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = (k >> 2) * (BT * 128) + (k & 3) * 32;
          umma_bf16_ss(tm_dPT, make_smem_desc(bdO + off, 16, 1024), make_smem_desc(aV + off, 16, 1024), idesc_s,
                       k > 0 ? 1u : 0u);
        }
        umma_commit(st_full);
        if (++st_s == Cfg::QS) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      auto issue_grads = [&](int t) {
        const int pb = Cfg::PDB ? (t & 1) : 0;
        const uint32_t aPT = smem_u32(sPT + pb * Cfg::PT_BYTES), adST = smem_u32(sdST + pb * Cfg::PT_BYTES);
        const uint32_t bQ = smem_u32(sQ + st_g * Cfg::T_BYTES), bdO = smem_u32(sdO + st_g * Cfg::T_BYTES);
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {   // k walks 16 query rows at a time in both operands
          umma_bf16_ss(tm_dV, make_smem_desc(aPT + k * (16 * 128), BT * 128, 1024),
                       make_smem_desc(bdO + k * (16 * 128), BT * 128, 1024), idesc_g, (t > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          umma_bf16_ss(tm_dK, make_smem_desc(adST + k * (16 * 128), BT * 128, 1024),
                       make_smem_desc(bQ + k * (16 * 128), BT * 128, 1024), idesc_g, (t > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&q_empty[st_g]);
        if (++st_g == Cfg::QS) st_g = 0;
      };
      if (ok && n_iter > 0) ok = issue_scores();
      for (int t = 0; t < n_iter && ok; ++t) {
        if (!mbar_wait(p_full, t & 1, p.status, ST_TIMEOUT_MISC)) { ok = false; break; }
        tc_fence_after();
        // scores of t+1 first (double-buffered P^T / dS^T): the softmax warps wait for nothing else, and the
        // commit of these scores also covers the gradient MMAs of t-1, which is what lets the softmax warps
        // reuse the P^T / dS^T buffer of parity (t+1)&1
        // (the dS store of t-1 has long been read out of its buffer; the wait only makes that certain before the
        // scores whose completion lets the softmax warps write that buffer again)
        if (p.spill_ds) tma_store_wait_read<0>();
        if (Cfg::PDB && t + 1 < n_iter) ok = issue_scores();
        if (p.spill_ds) {
          // the finished dS tile (bf16, [q rows][kv], scale included) also goes to global memory, where
          // the dQ kernel streams it back instead of recomputing scores; the bulk store reads shared
          // memory asynchronously, so it must have been read out before this buffer is written again
          const int head = kvh * group + t / n_qt;
          const int qt = qt_first + t % n_qt;
          const uint8_t* src = sdST + (Cfg::PDB ? (t & 1) : 0) * Cfg::PT_BYTES;
          tma_store_3d(&tm_ds, src, kv0, qt * BT, b * p.H + head);
          tma_store_3d(&tm_ds, src + BT * 128, kv0 + 64, qt * BT, b * p.H + head);
          tma_store_commit();
        }
        issue_grads(t);
        if (!Cfg::PDB) {
          if (p.spill_ds) tma_store_wait_read<0>();   // single dS buffer: read out before it is rewritten
          if (t + 1 < n_iter) ok = issue_scores();
        }
      }
      if (ok) umma_commit(done);
      if (p.spill_ds) tma_store_wait<0>();   // the stores are complete before the CTA retires
    }
  } else {
    const int sw = warp - 2;        // 0..7
    const int q = warp & 3;         // TMEM lane quarter
    const int half = sw >> 2;       // which 64 kv columns of the tile this warp handles
    const int r = q * 32 + lane;    // row inside the tile == TMEM lane (query row in the loop, kv row at the end)
    const int kv_idx = kv0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const float delta_scale = p.scale;
    bool ok = true;
    for (int t = 0; t < n_iter; ++t) {
      const int head = kvh * group + t / n_qt;
      const int qt = qt_first + t % n_qt;
      const int q0 = qt * BT;
      const int q_idx = q0 + r;
      const float2 sd = __ldg(p.stats + (static_cast<size_t>(b) * p.H + head) * p.S + min(q_idx, p.S - 1));
      const int pb = Cfg::PDB ? (t & 1) : 0;
      uint8_t* pt_buf = sPT + pb * Cfg::PT_BYTES;
      uint8_t* dst_buf = sdST + pb * Cfg::PT_BYTES;
      // last visible kv column of this query row inside the tile (-1: row is past the sequence end)
      const bool diag = p.causal && qt == kt;
      int lim = min(diag ? r : BT - 1, p.S - 1 - kv0);
      if (q_idx >= p.S) lim = -1;
      const bool need_mask = diag || (q0 + BT > p.S) || (kv0 + BT > p.S);
      if (!mbar_wait(st_full, t & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (need_mask) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
          bwd_chunk<true, true>(tm_ST, tm_dPT, lane_off, half * 2 + cc, r, lim, p.scale_log2, sd.x,
                                sd.y * delta_scale, p.scale, pt_buf, dst_buf);
      } else {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
          bwd_chunk<false, true>(tm_ST, tm_dPT, lane_off, half * 2 + cc, r, lim, p.scale_log2, sd.x,
                                 sd.y * delta_scale, p.scale, pt_buf, dst_buf);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(done, 0, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      constexpr int CPW = DH / 64;  // 32-column chunks per warp and matrix
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tm_dK : tm_dV;
        const int col0 = (which == 0 ? (p.H + kvh) : (p.H + p.Hkv + kvh)) * DH;
#pragma unroll 1
        for (int cc = 0; cc < CPW; ++cc) {
          const int c = half * CPW + cc;
          uint32_t v[32];
          tmem_ld_32x32(src + lane_off + c * 32, v);
          tmem_ld_wait();
          if (kv_idx < p.S) {
            __nv_bfloat16* dst = p.dqkv + static_cast<size_t>(row_base + kv_idx) * p.ld_dqkv + col0 + c * 32;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(v[u * 8 + 0]), __uint_as_float(v[u * 8 + 1]));
              w.y = pack_bf16x2(__uint_as_float(v[u * 8 + 2]), __uint_as_float(v[u * 8 + 3]));
              w.z = pack_bf16x2(__uint_as_float(v[u * 8 + 4]), __uint_as_float(v[u * 8 + 5]));
              w.w = pack_bf16x2(__uint_as_float(v[u * 8 + 6]), __uint_as_float(v[u * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + u * 8) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// --------------------------------------------------------------------------- dQ
template <int DH>
struct DqCfg {
  static constexpr bool PDB = (DH == 64);        // double-buffer dS
  static constexpr int NPB = PDB ? 2 : 1;
  static constexpr int KS = (DH == 64) ? 2 : 1;  // (K, V) ring stages
  static constexpr int T_BYTES = BT * DH * 2;
  static constexpr int DS_BYTES = BT * BT * 2;
  static constexpr int TILE_BYTES = 2 * T_BYTES + KS * 2 * T_BYTES + NPB * DS_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 1024 + 128;
  static constexpr int TMEM_COLS = 512;  // S 128 | dP 128 | dQ DH
};

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                        const BwdParams p) {
  using Cfg = DqCfg<DH>;
  constexpr int NCH = DH / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + Cfg::T_BYTES;
  uint8_t* sK = sdO + Cfg::T_BYTES;               // KS stages
  uint8_t* sV = sK + Cfg::KS * Cfg::T_BYTES;      // KS stages
  uint8_t* sdS = sV + Cfg::KS * Cfg::T_BYTES;     // NPB buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + Cfg::NPB * Cfg::DS_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;            // KS
  uint64_t* kv_empty = kv_full + Cfg::KS;  // KS
  uint64_t* s_full = kv_empty + Cfg::KS;
  uint64_t* p_full = s_full + 1;
  uint64_t* done = p_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (p.S + BT - 1) / BT;
  const int qt = n_t - 1 - blockIdx.z;   // slowest grid index: longest rows of tiles first over the whole grid
  const int head = blockIdx.x, b = blockIdx.y;
  const int kvh = head / (p.H / p.Hkv);
  const int q0 = qt * BT;
  const int row_base = b * p.S;
  const int n_blocks = p.causal ? (qt + 1) : n_t;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < Cfg::KS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(done, 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tm_qkv); prefetch_tmap(&tm_do); }
  if (warp == 1) { tmem_alloc(tmem_holder, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const uint32_t tm_S = tmem_base, tm_dP = tmem_base + 128, tm_dQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * Cfg::T_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tma_load_2d(sQ + c * (BT * 128), &tm_qkv, q_full, head * DH + c * 64, row_base + q0);
        tma_load_2d(sdO + c * (BT * 128), &tm_do, q_full, head * DH + c * 64, row_base + q0);
      }
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_blocks; ++j) {
        if (!mbar_wait(&kv_empty[st], ph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&kv_full[st], 2 * Cfg::T_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sK + st * Cfg::T_BYTES + c * (BT * 128), &tm_qkv, &kv_full[st], (p.H + kvh) * DH + c * 64,
                      row_base + j * BT);
          tma_load_2d(sV + st * Cfg::T_BYTES + c * (BT * 128), &tm_qkv, &kv_full[st],
                      (p.H + p.Hkv + kvh) * DH + c * 64, row_base + j * BT);
        }
        if (++st == Cfg::KS) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BT, BT, false, false);
      constexpr uint32_t idesc_g = make_idesc_bf16(BT, DH, false, true);
      bool ok = mbar_wait(q_full, 0, p.status, ST_TIMEOUT_FULL);
      int st_s = 0, st_g = 0;
      uint32_t ph_s = 0;
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO);
      auto issue_scores = [&]() -> bool {
        if (!mbar_wait(&kv_full[st_s], ph_s, p.status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t bK = smem_u32(sK + st_s * Cfg::T_BYTES), bV = smem_u32(sV + st_s * Cfg::T_BYTES);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = (k >> 2) * (BT * 128) + (k & 3) * 32;
          umma_bf16_ss(tm_S, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(bK + off, 16, 1024), idesc_s,
                       k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = (k >> 2) * (BT * 128) + (k & 3) * 32;
          umma_bf16_ss(tm_dP, make_smem_desc(adO + off, 16, 1024), make_smem_desc(bV + off, 16, 1024), idesc_s,
                       k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (++st_s == Cfg::KS) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      auto issue_grad = [&](int j) {
        const int pb = Cfg::PDB ? (j & 1) : 0;
        const uint32_t adS = smem_u32(sdS + pb * Cfg::DS_BYTES), bK = smem_u32(sK + st_g * Cfg::T_BYTES);
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t aoff = (k >> 2) * (BT * 128) + (k & 3) * 32;
          umma_bf16_ss(tm_dQ, make_smem_desc(adS + aoff, 16, 1024),
                       make_smem_desc(bK + k * (16 * 128), BT * 128, 1024), idesc_g, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[st_g]);
        if (++st_g == Cfg::KS) st_g = 0;
      };
      if (ok) ok = issue_scores();
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (!mbar_wait(p_full, j & 1, p.status, ST_TIMEOUT_MISC)) { ok = false; break; }
        tc_fence_after();
        if (Cfg::PDB) {
          if (j + 1 < n_blocks) ok = issue_scores();
          issue_grad(j);
        } else {
          issue_grad(j);
          if (j + 1 < n_blocks) ok = issue_scores();
        }
      }
      if (ok) umma_commit(done);
    }
  } else {
    const int sw = warp - 2;
    const int q = warp & 3;
    const int half = sw >> 2;
    const int r = q * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float lse2 = 0.f, del = 0.f;
    if (q_idx < p.S) {
      const float2 sd = p.stats[(static_cast<size_t>(b) * p.H + head) * p.S + q_idx];
      lse2 = sd.x;
      del = sd.y;
    }
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      if (!mbar_wait(s_full, j & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BT;
      const bool diag = p.causal && j == n_blocks - 1;
      const bool need_mask = diag || (kv0 + BT > p.S) || (q0 + BT > p.S);
      int lim = min(diag ? r : BT - 1, p.S - 1 - kv0);
      if (q_idx >= p.S) lim = -1;
      uint8_t* ds_buf = sdS + (Cfg::PDB ? (j & 1) : 0) * Cfg::DS_BYTES;
      if (need_mask) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
          bwd_chunk<true, false>(tm_S, tm_dP, lane_off, half * 2 + cc, r, lim, p.scale_log2, lse2, del * p.scale,
                                 p.scale, nullptr, ds_buf);
      } else {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
          bwd_chunk<false, false>(tm_S, tm_dP, lane_off, half * 2 + cc, r, lim, p.scale_log2, lse2, del * p.scale,
                                  p.scale, nullptr, ds_buf);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(done, 0, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      constexpr int CPW = DH / 64;
#pragma unroll 1
      for (int cc = 0; cc < CPW; ++cc) {
        const int c = half * CPW + cc;
        uint32_t v[32];
        tmem_ld_32x32(tm_dQ + lane_off + c * 32, v);
        tmem_ld_wait();
        if (q_idx < p.S) {
          __nv_bfloat16* dst = p.dqkv + static_cast<size_t>(row_base + q_idx) * p.ld_dqkv + head * DH + c * 32;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[u * 8 + 0]), __uint_as_float(v[u * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(v[u * 8 + 2]), __uint_as_float(v[u * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(v[u * 8 + 4]), __uint_as_float(v[u * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(v[u * 8 + 6]), __uint_as_float(v[u * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + u * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}


// --------------------------------------------------------------------------- dQ from stored dS
// When the dK/dV kernel has spilled its dS tiles (bf16 [B*H, S, S], scale included), dQ = dS K is a
// plain streamed product: no scores, no exponentials. One CTA per (query tile, head, batch) walks the
// kv tiles in ascending order through a TMA ring of (dS tile, K tile) pairs and accumulates in TMEM.
// It is bound by the bytes of dS (half of S x S per head under the causal mask).
template <int DH>
struct DqsCfg {
  static constexpr int DS_BYTES = BT * BT * 2;
  static constexpr int K_BYTES = BT * DH * 2;
  static constexpr int STAGE_BYTES = DS_BYTES + K_BYTES;
  static constexpr int STAGES = (DH == 64) ? 4 : 3;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 128;
  static constexpr int TMEM_COLS = DH;
};

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attention_bwd_dq_stream_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_ds,
                               const BwdParams p) {
  using Cfg = DqsCfg<DH>;
  constexpr int NCH = DH / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::STAGES;
  uint64_t* done = empty + Cfg::STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = (p.S + BT - 1) / BT;
  const int qt = n_t - 1 - blockIdx.z;   // slowest grid index: longest rows of tiles first over the whole grid
  const int head = blockIdx.x, b = blockIdx.y;
  const int kvh = head / (p.H / p.Hkv);
  const int q0 = qt * BT;
  const int row_base = b * p.S;
  const int n_blocks = p.causal ? (qt + 1) : n_t;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(done, 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tm_qkv); prefetch_tmap(&tm_ds); }
  if (warp == 1) { tmem_alloc(tmem_holder, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm_dQ = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    if (lane == 0) {
      int st = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_blocks; ++j) {
        if (!mbar_wait(&empty[st], ph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        uint8_t* sdS = smem + st * Cfg::STAGE_BYTES;
        uint8_t* sK = sdS + Cfg::DS_BYTES;
        mbar_arrive_expect_tx(&full[st], Cfg::STAGE_BYTES);
        tma_load_3d(sdS, &tm_ds, &full[st], j * BT, q0, b * p.H + head);
        tma_load_3d(sdS + BT * 128, &tm_ds, &full[st], j * BT + 64, q0, b * p.H + head);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sK + c * (BT * 128), &tm_qkv, &full[st], (p.H + kvh) * DH + c * 64, row_base + j * BT);
        if (++st == Cfg::STAGES) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_g = make_idesc_bf16(BT, DH, false, true);
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (!mbar_wait(&full[st], ph, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t adS = smem_u32(smem + st * Cfg::STAGE_BYTES), bK = adS + Cfg::DS_BYTES;
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t aoff = (k >> 2) * (BT * 128) + (k & 3) * 32;
          umma_bf16_ss(tm_dQ, make_smem_desc(adS + aoff, 16, 1024), make_smem_desc(bK + k * (16 * 128), BT * 128, 1024),
                       idesc_g, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty[st]);
        if (++st == Cfg::STAGES) { st = 0; ph ^= 1; }
      }
      if (ok) umma_commit(done);
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    if (mbar_wait(done, 0, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      constexpr int CPW = DH / 64;
#pragma unroll 1
      for (int cc = 0; cc < CPW; ++cc) {
        const int c = half * CPW + cc;
        uint32_t v[32];
        tmem_ld_32x32(tm_dQ + lane_off + c * 32, v);
        tmem_ld_wait();
        if (q_idx < p.S) {
          __nv_bfloat16* dst = p.dqkv + static_cast<size_t>(row_base + q_idx) * p.ld_dqkv + head * DH + c * 32;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[u * 8 + 0]), __uint_as_float(v[u * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(v[u * 8 + 2]), __uint_as_float(v[u * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(v[u * 8 + 4]), __uint_as_float(v[u * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(v[u * 8 + 6]), __uint_as_float(v[u * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + u * 8) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tm_dQ, Cfg::TMEM_COLS);
}

template <int DH>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& td, const CUtensorMap& tds, const BwdParams& p,
                      cudaStream_t stream) {
  auto k1 = attention_bwd_dkv_kernel<DH>;
  auto k2 = attention_bwd_dq_kernel<DH>;
  auto k3 = attention_bwd_dq_stream_kernel<DH>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<DH>::SMEM_BYTES) !=
            cudaSuccess ||
        cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<DH>::SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, DqsCfg<DH>::SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  const int n_t = (p.S + BT - 1) / BT;
  k1<<<dim3(p.Hkv, p.B, n_t), BWD_THREADS, DkvCfg<DH>::SMEM_BYTES, stream>>>(tq, td, tds, p);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  if (p.spill_ds) k3<<<dim3(p.H, p.B, n_t), BWD_THREADS, DqsCfg<DH>::SMEM_BYTES, stream>>>(tq, tds, p);
  else k2<<<dim3(p.H, p.B, n_t), BWD_THREADS, DqCfg<DH>::SMEM_BYTES, stream>>>(tq, td, p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

using namespace sb;

// qkv, dqkv: bf16 [B*S, ld]; O, dO: bf16 [B*S, ld_o / ld_do] (H*dh columns); lse: fp32 [B,H,S];
// delta: scratch of 2*B*H*S floats written here ((lse*log2e, delta) pairs). dqkv receives dQ | dK | dV in
// the qkv layout. ds_scratch (optional): B*H*S*round_up(S, 64) bf16; with it the dK/dV kernel stores its
// dS tiles there and dQ is computed by streaming them back (faster: no second pass over the scores);
// without it dQ recomputes scores and exponentials.
extern "C" size_t sb_attention_bwd_ds_elems(int B, int S, int H) {
  return static_cast<size_t>(B) * H * S * ((S + 63) / 64 * 64);
}

extern "C" int sb_attention_bwd(const void* qkv, const void* O, const float* lse, const void* dO, void* dqkv,
                                float* delta, void* ds_scratch, int B, int S, int H, int Hkv, int dh, int ld,
                                int ld_o, int ld_do, float scale, int causal, int* status, void* stream_) {
  if (B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) || (dh != 64 && dh != 128)) return SB_ERR_ARG;
  if (B > 65535 || (S + 127) / 128 > 65535) return SB_ERR_TOO_LARGE;   // grid y / z limits
  if ((ld & 7) || (reinterpret_cast<uintptr_t>(dqkv) & 15)) return SB_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  CUtensorMap tq, td;
  int rc = make_tmap_2d_bf16(&tq, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(B) * S, ld, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&td, dO, static_cast<uint64_t>(H) * dh, static_cast<uint64_t>(B) * S, ld_do, 64, 128);
  if (rc) return rc;
  if ((ld_o & 7) || (ld_do & 7) || (reinterpret_cast<uintptr_t>(O) & 15) || (reinterpret_cast<uintptr_t>(dO) & 15))
    return SB_ERR_ALIGN;
  const long long groups = static_cast<long long>(B) * S * H;
  const int gpw = 32 / (dh / 8);
  const long long warps = (groups + gpw - 1) / gpw;
  attn_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(O),
                                                         static_cast<const __nv_bfloat16*>(dO), lse,
                                                         reinterpret_cast<float2*>(delta), B, S, H, dh, ld_o,
                                                         ld_do);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  BwdParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.ld_dqkv = ld;
  p.scale = scale;
  p.scale_log2 = scale * LOG2E;
  p.causal = causal;
  p.lse = lse;
  p.stats = reinterpret_cast<const float2*>(delta);
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.status = status;
  p.spill_ds = ds_scratch ? 1 : 0;
  CUtensorMap tds = tq;   // placeholder when unused
  if (ds_scratch) {
    const uint64_t sp = (static_cast<uint64_t>(S) + 63) / 64 * 64;
    rc = make_tmap_3d_bf16(&tds, ds_scratch, S, S, static_cast<uint64_t>(B) * H, sp, sp * S, 64, 128);
    if (rc) return rc;
  }
  return dh == 64 ? launch_bwd<64>(tq, td, tds, p, stream) : launch_bwd<128>(tq, td, tds, p, stream);
}
