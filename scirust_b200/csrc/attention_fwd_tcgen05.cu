// GQA flash-attention forward for sm_100a (prefill and training): S = Q K^T and O += P V on
// tcgen05 tensor cores with the accumulators in tensor memory, K/V/Q tiles brought in by TMA,
// online softmax in registers (one thread owns one query row, so no shuffles).
//
// Replaces the reference's per-(sequence, head) cuBLASLt GEMM pair plus scale_mask and
// softmax kernels, which materialise the S x S score matrix
// (scirust-sciagent/src/cuda_model.rs:796-832; scirust-cuda/src/chain.rs:168-222,448).
// Semantics: scores scaled by 1/sqrt(dh), causal mask j > i, fp32 softmax, bf16 P for the
// second product. KV blocks are visited in ascending order: results are bitwise repeatable.
//
// Layout: one fused activation matrix qkv [B*S, ld] (row = token) holding the RoPE'd q heads,
// then the k heads, then the v heads; query head h uses kv head h / (H / Hkv).
// Output O [B*S, H*dh] bf16 and LSE [B, H, S] fp32 (natural log) for the backward pass.
//
// CTA = (128-query tile, head, batch); 6 warps: 0 TMA producer, 1 MMA issuer, 2-5 softmax.
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

constexpr int ATT_BM = 128;  // query rows per CTA
constexpr int ATT_BN = 128;  // kv rows per block
constexpr int ATT_THREADS = 192;

template <int DH>
struct AttCfg {
  static constexpr int KS = 2;                      // K ring stages
  static constexpr int VS = (DH == 64) ? 1 : 2;     // V ring stages
  static constexpr int Q_BYTES = ATT_BM * DH * 2;
  static constexpr int KV_BYTES = ATT_BN * DH * 2;
  static constexpr int P_BYTES = ATT_BM * ATT_BN * 2;
  static constexpr int TILE_BYTES = Q_BYTES + (KS + VS) * KV_BYTES + P_BYTES;
  static constexpr int SMEM_BYTES = TILE_BYTES + 1024 + 128;
  static constexpr int TMEM_COLS = 256;             // S: 128 columns, O block: DH columns
};

struct AttParams {
  int B, S, H, Hkv;
  int ld_o;
  float scale_log2;  // (1/sqrt(dh)) * log2(e)
  int causal;
  __nv_bfloat16* O;
  float* lse;
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Online-softmax update for one 128-column score block of one query row (thread = row r = TMEM
// lane): pass 1 finds the row maximum, pass 2 writes P = 2^(s*sl2 - m_new) as bf16 into the
// 128B-swizzled K-major tile and sums it. `m` is updated; alpha = 2^(m_old - m_new).
template <bool MASK>
__device__ __forceinline__ void softmax_block(uint32_t taddr, uint8_t* sP, int r, int lim, float sl2, float& m,
                                              float& alpha, float& rowsum) {
  constexpr float NEG = -1.0e30f;
  float mx = NEG;
#pragma unroll 1
  for (int c = 0; c < ATT_BN / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c * 32, v);
    tmem_ld_wait();
    float m4[4] = {NEG, NEG, NEG, NEG};   // four chains shorten the dependency chain of the max
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float s = __uint_as_float(v[i]);
      if (MASK && c * 32 + i > lim) s = NEG;
      m4[i & 3] = fmaxf(m4[i & 3], s);
    }
    mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
  }
  const float m_new = fmaxf(m, mx * sl2);
  alpha = fast_exp2(m - m_new);
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
  for (int c = 0; c < ATT_BN / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c * 32, v);
    tmem_ld_wait();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -m_new));
      float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), sl2, -m_new));
      if (MASK) {
        if (c * 32 + i > lim) p0 = 0.f;
        if (c * 32 + i + 1 > lim) p1 = 0.f;
      }
      sum4[(i >> 1) & 3] += p0 + p1;
      pk[i >> 1] = pack_bf16x2(p0, p1);
    }
    uint8_t* prow = sP + (c >> 1) * (ATT_BM * 128) + r * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int unit = ((c & 1) * 4 + u) ^ (r & 7);
      *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
    }
  }
  rowsum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
  m = m_new;
}

template <int DH>
__global__ void __launch_bounds__(ATT_THREADS)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap, const AttParams p) {
  using Cfg = AttCfg<DH>;
  constexpr int NCH = DH / 64;  // 64-column chunks per head
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;
  uint8_t* sV = sK + Cfg::KS * Cfg::KV_BYTES;
  uint8_t* sP = sV + Cfg::VS * Cfg::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + Cfg::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + Cfg::KS;
  uint64_t* v_full = k_empty + Cfg::KS;
  uint64_t* v_empty = v_full + Cfg::VS;
  uint64_t* s_full = v_empty + Cfg::VS;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = p_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + ATT_BM - 1) / ATT_BM;
  const int qt = n_qt - 1 - blockIdx.z;  // slowest grid index: longest (most kv blocks) tiles first over the whole grid
  const int head = blockIdx.x, b = blockIdx.y;
  const int kvh = head / (p.H / p.Hkv);
  const int q0 = qt * ATT_BM;
  const int row_base = b * p.S;
  const int n_blocks = p.causal ? (qt + 1) : (p.S + ATT_BN - 1) / ATT_BN;
  const int col_q = head * DH;
  const int col_k = (p.H + kvh) * DH;
  const int col_v = (p.H + p.Hkv + kvh) * DH;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < Cfg::KS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < Cfg::VS; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) prefetch_tmap(&tmap);
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c)
        tma_load_2d(sQ + c * (ATT_BM * 128), &tmap, q_full, col_q + c * 64, row_base + q0);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      for (int j = 0; j < n_blocks; ++j) {
        const int r = row_base + j * ATT_BN;
        if (!mbar_wait(&k_empty[ks], kph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&k_full[ks], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sK + ks * Cfg::KV_BYTES + c * (ATT_BN * 128), &tmap, &k_full[ks], col_k + c * 64, r);
        if (++ks == Cfg::KS) { ks = 0; kph ^= 1; }
        if (!mbar_wait(&v_empty[vs], vph ^ 1, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_arrive_expect_tx(&v_full[vs], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sV + vs * Cfg::KV_BYTES + c * (ATT_BN * 128), &tmap, &v_full[vs], col_v + c * 64, r);
        if (++vs == Cfg::VS) { vs = 0; vph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(ATT_BM, DH, false, true);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      bool ok = mbar_wait(q_full, 0, p.status, ST_TIMEOUT_FULL);
      auto issue_s = [&]() -> bool {
        if (!mbar_wait(&k_full[ks], kph, p.status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK + ks * Cfg::KV_BYTES);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k) {
          const uint32_t off = (k >> 2) * (ATT_BM * 128) + (k & 3) * 32;
          umma_bf16_ss(tmem_S, make_smem_desc(aq + off, 16, 1024), make_smem_desc(bk + off, 16, 1024), idesc_s,
                       k > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[ks]);
        umma_commit(s_full);
        if (++ks == Cfg::KS) { ks = 0; kph ^= 1; }
        return true;
      };
      if (ok) ok = issue_s();
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (!mbar_wait(p_full, j & 1, p.status, ST_TIMEOUT_MISC)) break;
        if (!mbar_wait(&v_full[vs], vph, p.status, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        const uint32_t ap = smem_u32(sP), bv = smem_u32(sV + vs * Cfg::KV_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          const uint64_t adesc = make_smem_desc(ap + (k >> 2) * (ATT_BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(bv + k * (16 * 128), ATT_BN * 128, 1024);
          umma_bf16_ss(tmem_O, adesc, bdesc, idesc_o, k > 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[vs]);
        umma_commit(o_full);
        if (++vs == Cfg::VS) { vs = 0; vph ^= 1; }
        if (j + 1 < n_blocks) ok = issue_s();
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;       // row inside the tile == TMEM lane
    const int q_idx = q0 + r;          // position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    constexpr float NEG = -1.0e30f;
    float m = NEG, l = 0.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      if (!mbar_wait(s_full, j & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * ATT_BN;
      const bool need_mask = (p.causal && j == n_blocks - 1) || (kv0 + ATT_BN > p.S);
      // last visible kv column of this row inside the block
      const int lim = (p.causal ? min(q_idx, p.S - 1) : (p.S - 1)) - kv0;
      float alpha, rowsum;
      if (need_mask) softmax_block<true>(tmem_S + lane_off, sP, r, lim, p.scale_log2, m, alpha, rowsum);
      else softmax_block<false>(tmem_S + lane_off, sP, r, lim, p.scale_log2, m, alpha, rowsum);
      l = l * alpha + rowsum;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!mbar_wait(o_full, j & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
    }
    if (ok && q_idx < p.S) {
      const float inv_l = 1.f / l;
      __nv_bfloat16* orow = p.O + static_cast<size_t>(row_base + q_idx) * p.ld_o + head * DH;
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        uint4 w;
        w.x = pack_bf16x2(o[c * 8 + 0] * inv_l, o[c * 8 + 1] * inv_l);
        w.y = pack_bf16x2(o[c * 8 + 2] * inv_l, o[c * 8 + 3] * inv_l);
        w.z = pack_bf16x2(o[c * 8 + 4] * inv_l, o[c * 8 + 5] * inv_l);
        w.w = pack_bf16x2(o[c * 8 + 6] * inv_l, o[c * 8 + 7] * inv_l);
        *reinterpret_cast<uint4*>(orow + c * 8) = w;
      }
      if (p.lse) p.lse[(static_cast<size_t>(b) * p.H + head) * p.S + q_idx] = m * 0.6931471805599453f + logf(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int DH>
static int launch_att_fwd(const CUtensorMap& tm, const AttParams& p, cudaStream_t stream) {
  using Cfg = AttCfg<DH>;
  auto kern = attention_fwd_kernel<DH>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  dim3 grid(p.H, p.B, (p.S + ATT_BM - 1) / ATT_BM);
  kern<<<grid, ATT_THREADS, Cfg::SMEM_BYTES, stream>>>(tm, p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

using namespace sb;

// qkv: bf16 [B*S, ld] = [q heads | k heads | v heads]; O: bf16 [B*S, ld_o]; lse: fp32 [B,H,S] or null.
extern "C" int sb_attention_fwd(const void* qkv, void* O, float* lse, int B, int S, int H, int Hkv, int dh, int ld,
                                int ld_o, float scale, int causal, int* status, void* stream_) {
  if (B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) || (dh != 64 && dh != 128)) return SB_ERR_ARG;
  if (B > 65535 || (S + 127) / 128 > 65535) return SB_ERR_TOO_LARGE;   // grid y / z limits
  if ((ld_o & 7) || (reinterpret_cast<uintptr_t>(O) & 15)) return SB_ERR_ALIGN;
  CUtensorMap tm;
  int rc = make_tmap_2d_bf16(&tm, qkv, static_cast<uint64_t>(ld), static_cast<uint64_t>(B) * S, ld, 64, 128);
  if (rc) return rc;
  AttParams p;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.ld_o = ld_o;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.O = static_cast<__nv_bfloat16*>(O);
  p.lse = lse;
  p.status = status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  return dh == 64 ? launch_att_fwd<64>(tm, p, stream) : launch_att_fwd<128>(tm, p, stream);
}
