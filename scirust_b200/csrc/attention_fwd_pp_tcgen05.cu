// GQA flash-attention forward for sm_100a, head dimension 64, two query tiles per CTA.
//
// One CTA owns 256 query rows of one (head, batch) as two 128-row tiles. Each tile has its own
// score accumulator S_t and output accumulator O_t in tensor memory and its own group of four
// softmax warps, so while the warps of one tile run their exponentials the tensor cores work on
// the other tile's products. The output accumulator stays in tensor memory for the whole loop:
// P V is accumulated there by the MMA itself, and a row is rescaled only when its running maximum
// has grown by more than 2^8 since the reference point used in the exponent (bf16 P then stays
// below 2^8, far inside its range), which on real score distributions happens in the first blocks
// only. The row sum uses the same reference point, so the final O / l and the log-sum-exp are
// exact regardless of when a rescale happened.
//
// Same interface, layout and semantics as the one-tile kernel (attention_fwd_tcgen05.cu): fused
// activation matrix qkv [B*S, ld] = [q heads | k heads | v heads], scores scaled by 1/sqrt(dh),
// causal mask j > i, fp32 softmax, bf16 P, O [B*S, H*dh] bf16, LSE [B, H, S] fp32. KV blocks are
// visited in ascending order and every decision depends on the data only, so results are bitwise
// repeatable. Counterpart in the reference: the per-(sequence, head) GEMM + scale_mask + softmax
// chain of scirust-sciagent/src/cuda_model.rs:796-832.
//
// A softmax thread holds its whole 128-column score row in registers (one pass over tensor memory),
// scales it with packed fp32 pairs (fma.rn.f32x2, add.rn.f32x2: half the issue slots of scalar
// code) and takes the row maximum with three-input max. Cycle stamps taken inside the kernel put a kv
// block of one tile at about 3500 cycles: 1500-1650 in the 128 exponentials with pack and store,
// 400 in the row maximum, and about 1000 waiting for the tensor pipe (scores of the next block, P V
// of the previous one), although the products themselves need only 256 + 436 cycles (a 128 x 128 x 16
// tcgen05.mma takes 64 cycles, a 128 x 64 x 16 one 54.5: `bench_kernels umma`). Two variants that
// looked right on paper measured slower and are not used: issuing the scores of block j+1 as soon
// as block j sits in registers (the P V of block j then queued behind them), and taking every
// fourth 2^x from a cubic polynomial on the FMA pipe (POLY_EVERY below; the softmax warps are short
// of issue slots per warp, not of special-function throughput).
//
// Warps: 0 TMA producer, 1 MMA issuer, 2-5 softmax of tile 0, 6-9 softmax of tile 1.
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

namespace attpp {

constexpr int BM = 128;        // query rows per tile
constexpr int BN = 128;        // kv rows per block
constexpr int DH = 64;
constexpr int THREADS = 320;
constexpr int KS = 3, VS = 3;  // K / V ring stages
constexpr int Q_BYTES = BM * DH * 2;
constexpr int KV_BYTES = BN * DH * 2;
constexpr int P_BYTES = BM * BN * 2;
constexpr int TILE_BYTES = 2 * Q_BYTES + (KS + VS) * KV_BYTES + 2 * P_BYTES;
constexpr int SMEM_BYTES = TILE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;  // S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384)
constexpr float RESCALE_GAP = 8.f;

struct Params {
  int B, S, H, Hkv;
  int ld_o;
  float scale_log2;  // (1/sqrt(dh)) * log2(e)
  int causal;
  __nv_bfloat16* O;
  float* lse;
  int* status;
};

constexpr int POLY_EVERY = 0;   // every POLY_EVERY-th element takes 2^x from the polynomial (0 = none)

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA pipe: n = round(x), f = x - n in [-0.5, 0.5], cubic minimax polynomial for 2^f,
// n added to the exponent field. x is clamped at -126 (the result is then about 1e-38).
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float magic = 12582912.f;            // 1.5 * 2^23: the sum holds round(x) in its low mantissa bits
  const float xr = x + magic;
  const float f = x - (xr - magic);
  float pl = fmaf(0.0551716685295105f, f, 0.2426111251115799f);
  pl = fmaf(pl, f, 0.6932609677314758f);
  pl = fmaf(pl, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(xr) << 23));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__global__ void __launch_bounds__(THREADS, 1)
attention_fwd_pp_kernel(const __grid_constant__ CUtensorMap tmap, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + 2 * Q_BYTES;
  uint8_t* sV = sK + KS * KV_BYTES;
  uint8_t* sP = sV + VS * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * P_BYTES);
  uint64_t* q_full = bars;               // [2]
  uint64_t* k_full = q_full + 2;         // [KS]
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;       // [VS]
  uint64_t* v_empty = v_full + VS;
  uint64_t* s_full = v_empty + VS;       // [2] scores of tile t are in tensor memory
  uint64_t* p_full = s_full + 2;         // [2] P of tile t is in shared memory (4 warp arrivals)
  uint64_t* pv_done = p_full + 2;        // [2] P V of tile t has completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_pairs = (p.S + 2 * BM - 1) / (2 * BM);
  const int pair = n_pairs - 1 - blockIdx.z;  // slowest grid index: longest tiles first over the whole grid
  const int head = blockIdx.x, b = blockIdx.y;
  const int kvh = head / (p.H / p.Hkv);
  const int q0 = pair * 2 * BM;
  const int row_base = b * p.S;
  const int nkv = (p.S + BN - 1) / BN;
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0t = q0 + t * BM;
    nb[t] = q0t >= p.S ? 0 : (p.causal ? min(q0t / BN + 1, nkv) : nkv);
  }
  const int n_blocks = max(nb[0], nb[1]);
  const int col_q = head * DH;
  const int col_k = (p.H + kvh) * DH;
  const int col_v = (p.H + p.Hkv + kvh) * DH;

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&pv_done[t], 1);
    }
    for (int s = 0; s < KS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < VS; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) prefetch_tmap(&tmap);
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ------------------------------------ TMA producer ------------------------------------
    if (lane == 0) {
      for (int t = 0; t < 2; ++t) {
        if (nb[t] > 0) {
          mbar_arrive_expect_tx(&q_full[t], Q_BYTES);
          tma_load_2d(sQ + t * Q_BYTES, &tmap, &q_full[t], col_q, row_base + q0 + t * BM);
        }
      }
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      for (int j = 0; j < n_blocks; ++j) {
        const int r = row_base + j * BN;
        if (!mbar_wait(&k_empty[ks], kph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&k_full[ks], KV_BYTES);
        tma_load_2d(sK + ks * KV_BYTES, &tmap, &k_full[ks], col_k, r);
        if (++ks == KS) { ks = 0; kph ^= 1; }
        if (!mbar_wait(&v_empty[vs], vph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&v_full[vs], KV_BYTES);
        tma_load_2d(sV + vs * KV_BYTES, &tmap, &v_full[vs], col_v, r);
        if (++vs == VS) { vs = 0; vph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------- MMA issuer -------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, DH, false, true);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      bool ok = true;
      for (int t = 0; t < 2 && ok; ++t)
        if (nb[t] > 0) ok = mbar_wait(&q_full[t], 0, p.status, ST_TIMEOUT_FULL);
      // S_t = Q_t K^T with K in ring slot `slot`
      auto issue_s = [&](int t, int slot) {
        const uint32_t aq = smem_u32(sQ + t * Q_BYTES), bk = smem_u32(sK + slot * KV_BYTES);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          umma_bf16_ss(tmem_base + t * BN, make_smem_desc(aq + k * 32, 16, 1024), make_smem_desc(bk + k * 32, 16, 1024),
                       idesc_s, k > 0 ? 1u : 0u);
        umma_commit(&s_full[t]);
      };
      // O_t (+)= P_t V with V in ring slot `slot`
      auto issue_pv = [&](int t, int slot, bool acc) {
        const uint32_t ap = smem_u32(sP + t * P_BYTES), bv = smem_u32(sV + slot * KV_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t adesc = make_smem_desc(ap + (k >> 2) * (BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(bv + k * (16 * 128), BN * 128, 1024);
          umma_bf16_ss(tmem_base + 2 * BN + t * DH, adesc, bdesc, idesc_o, (acc || k > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[t]);
      };
      if (ok && n_blocks > 0) {
        ok = mbar_wait(&k_full[ks], kph, p.status, ST_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after();
          for (int t = 0; t < 2; ++t)
            if (nb[t] > 0) issue_s(t, ks);
          umma_commit(&k_empty[ks]);
          if (++ks == KS) { ks = 0; kph ^= 1; }
        }
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const bool have_next = j + 1 < n_blocks;
        if (have_next && !mbar_wait(&k_full[ks], kph, p.status, ST_TIMEOUT_FULL)) break;
        if (!mbar_wait(&v_full[vs], vph, p.status, ST_TIMEOUT_FULL)) break;
        for (int t = 0; t < 2; ++t) {
          if (j >= nb[t]) continue;
          if (!mbar_wait(&p_full[t], j & 1, p.status, ST_TIMEOUT_MISC)) { ok = false; break; }
          tc_fence_after();
          if (j + 1 < nb[t]) issue_s(t, ks);   // scores first: the softmax warps of this tile can go on
          issue_pv(t, vs, j > 0);
        }
        if (!ok) break;
        if (have_next) {
          umma_commit(&k_empty[ks]);
          if (++ks == KS) { ks = 0; kph ^= 1; }
        }
        umma_commit(&v_empty[vs]);
        if (++vs == VS) { vs = 0; vph ^= 1; }
      }
    }
  } else {
    // ------------------------------------ softmax warps ------------------------------------
    const int t = (warp - 2) >> 2;
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;       // row inside the tile == TMEM lane
    const int q_idx = q0 + t * BM + r; // position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t tm_S = tmem_base + t * BN + lane_off;
    const uint32_t tm_O = tmem_base + 2 * BN + t * DH + lane_off;
    uint8_t* sPt = sP + t * P_BYTES;
    const float sl2 = p.scale_log2;
    constexpr float NEG = -1.0e30f;
    float m_ref = NEG, l = 0.f;
    bool ok = true;
    const int n_t = nb[t];
    for (int j = 0; j < n_t; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld_32x32(tm_S + c * 32, v + c * 32);
      tmem_ld_wait();
      const int kv0 = j * BN;
      const bool need_mask = (p.causal && j == n_t - 1) || (kv0 + BN > p.S);
      const int lim = (p.causal ? min(q_idx, p.S - 1) : (p.S - 1)) - kv0;   // last visible column
      float m4[4] = {NEG, NEG, NEG, NEG};
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BN; i += 2)
          m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], i > lim ? NEG : __uint_as_float(v[i]),
                                  i + 1 > lim ? NEG : __uint_as_float(v[i + 1]));
      } else {
#pragma unroll
        for (int i = 0; i < BN; i += 2)
          m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      }
      const float m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl2;
      const bool grow = m_blk > m_ref + RESCALE_GAP;   // always true in the first block
      if (j > 0) {
        // P V of the previous block has read the P tile and updated O
        if (!mbar_wait(&pv_done[t], (j - 1) & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        if (__any_sync(0xffffffffu, grow)) {
          tc_fence_after();
          const float alpha = grow ? ex2(m_ref - m_blk) : 1.f;
#pragma unroll
          for (int c = 0; c < DH / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(tm_O + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(tm_O + c * 16, o);
          }
          tmem_st_wait();
          l *= alpha;
        }
      }
      if (grow) m_ref = m_blk;
      // exponentials in place: every result lands in the register of its score, so all 128 are independent
      const float neg_m = -m_ref;
#pragma unroll
      for (int i = 0; i < BN; i += 2) {
        fma2(v[i], v[i + 1], sl2, neg_m);
        float e0 = (POLY_EVERY > 0 && (i % (POLY_EVERY > 0 ? POLY_EVERY : 1)) == POLY_EVERY - 1)
                       ? ex2_poly(__uint_as_float(v[i])) : ex2(__uint_as_float(v[i]));
        float e1 = (POLY_EVERY > 0 && ((i + 1) % (POLY_EVERY > 0 ? POLY_EVERY : 1)) == POLY_EVERY - 1)
                       ? ex2_poly(__uint_as_float(v[i + 1])) : ex2(__uint_as_float(v[i + 1]));
        if (need_mask) {
          if (i > lim) e0 = 0.f;
          if (i + 1 > lim) e1 = 0.f;
        }
        v[i] = __float_as_uint(e0);
        v[i + 1] = __float_as_uint(e1);
      }
      float sum4[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BN / 16; ++c) {          // 16 columns = two 16-byte units of the swizzled row
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          add2(sum4[i & 6], sum4[(i & 6) + 1], v[c * 16 + i], v[c * 16 + i + 1]);
          pk[i >> 1] = pack_bf16x2(__uint_as_float(v[c * 16 + i]), __uint_as_float(v[c * 16 + i + 1]));
        }
        uint8_t* prow = sPt + (c >> 2) * (BM * 128) + r * 128;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int unit = ((c & 3) * 2 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
        }
      }
      l += ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3])) + ((sum4[4] + sum4[5]) + (sum4[6] + sum4[7]));
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (ok && n_t > 0) ok = mbar_wait(&pv_done[t], (n_t - 1) & 1, p.status, ST_TIMEOUT_TMEM_FULL);
    if (ok && n_t > 0) {
      tc_fence_after();
      uint32_t o[DH];
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) tmem_ld_32x32(tm_O + c * 32, o + c * 32);
      tmem_ld_wait();
      if (q_idx < p.S) {
        const float inv_l = 1.f / l;
        __nv_bfloat16* orow = p.O + static_cast<size_t>(row_base + q_idx) * p.ld_o + head * DH;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[c * 8 + 0]) * inv_l, __uint_as_float(o[c * 8 + 1]) * inv_l);
          w.y = pack_bf16x2(__uint_as_float(o[c * 8 + 2]) * inv_l, __uint_as_float(o[c * 8 + 3]) * inv_l);
          w.z = pack_bf16x2(__uint_as_float(o[c * 8 + 4]) * inv_l, __uint_as_float(o[c * 8 + 5]) * inv_l);
          w.w = pack_bf16x2(__uint_as_float(o[c * 8 + 6]) * inv_l, __uint_as_float(o[c * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 8) = w;
        }
        if (p.lse) p.lse[(static_cast<size_t>(b) * p.H + head) * p.S + q_idx] = m_ref * 0.6931471805599453f + logf(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace attpp
}  // namespace sb

using namespace sb;

// Same arguments as sb_attention_fwd; head dimension 64 only.
extern "C" int sb_attention_fwd_pp(const void* qkv, void* O, float* lse, int B, int S, int H, int Hkv, int dh, int ld,
                                   int ld_o, float scale, int causal, int* status, void* stream_) {
  if (B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) || dh != attpp::DH) return SB_ERR_ARG;
  if (B > 65535 || (S + 127) / 128 > 65535) return SB_ERR_TOO_LARGE;   // grid y / z limits
  if ((ld_o & 7) || (reinterpret_cast<uintptr_t>(O) & 15)) return SB_ERR_ALIGN;
  CUtensorMap tm;
  int rc = make_tmap_2d_bf16(&tm, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(B) * S, ld, 64, 128);
  if (rc) return rc;
  attpp::Params p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.ld_o = ld_o;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.O = static_cast<__nv_bfloat16*>(O);
  p.lse = lse;
  p.status = status;
  auto kern = attpp::attention_fwd_pp_kernel;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, attpp::SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  dim3 grid(H, B, (S + 2 * attpp::BM - 1) / (2 * attpp::BM));
  kern<<<grid, attpp::THREADS, attpp::SMEM_BYTES, static_cast<cudaStream_t>(stream_)>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
