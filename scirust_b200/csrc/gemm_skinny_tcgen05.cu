// Weight-streaming GEMM for batched decoding: C[rows, N] = X[rows, K] . W (+ R) with 9..64 activation rows.
//
// With so few rows the product is bound by the weight bytes, and on this GPU a copy only reaches the HBM rate with
// about 30 MB in flight (the loaded latency is several microseconds). The general GEMM spends its shared memory on
// 128-row activation tiles that are mostly zero fill and keeps 128 KB of weights in flight per SM; here the roles are
// swapped: the WEIGHT tile is the 128-row MMA operand (128 output columns x one k-block, 16 KB), the activations
// are the narrow operand (16 / 32 / 64 rows x one k-block, 2-8 KB), so 9 to 12 stages fit (144-192 KB of weights in
// flight per SM) and every weight byte is read exactly once. The accumulator is C^T (lane = output column, TMEM
// column = activation row); the epilogue writes it back transposed.
//
//   bf16 (I8 = false): W [K, N] as stored (N contiguous) is the MN-major A operand, X [rows, K] the K-major B
//                      operand; tcgen05.mma.kind::f16, fp32 accumulation, k walked in ascending order.
//   int8 (I8 = true):  W8A8 of the reference's quantised linear layer (scirust-core/src/quantization.rs:150-190):
//                      weights as the transposed codes [N, K], activations quantised per row; kind::i8, int32
//                      accumulation (exact), one rescale by sx[m] * sw[n].
// Split-K partials (fp32 / int32, [split][row][N]) are added in split order by skinny_reduce_kernel.
// Warps: 0 TMA, 1 MMA, 2-5 epilogue (one per TMEM lane quarter).
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int num_sms();

constexpr int SK_BM = 128;          // output columns per tile (the MMA's M)
constexpr int SK_THREADS = 192;
constexpr int SK_A_BYTES = 16384;   // 128 columns x (64 bf16 | 128 int8) of k

template <int RB>
struct SkinnyCfg {
  static constexpr int B_BYTES = RB * 128;
  static constexpr int STAGE_BYTES = SK_A_BYTES + B_BYTES;
  static constexpr int STAGES = (227 * 1024 - 1280) / STAGE_BYTES;
  static constexpr int ACC_STRIDE = RB < 32 ? 32 : RB;       // TMEM columns between the two accumulators
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

struct SkinnyParams {
  int rows, N, K;
  int splits, kb_per_split;
  void* C; int ldc;               // bf16 [rows, ldc]; or partials [splits][rows][N] (fp32 / int32)
  const void* R; int ldr;
  const float* sx; const float* sw;   // int8 only
  int* status;
};

__host__ __device__ constexpr uint32_t skinny_idesc(bool i8, int n) {
  // kind::f16: D f32 (1 << 4), A / B bf16 (1 << 7, 1 << 10), A MN-major (1 << 15);  kind::i8: D s32 (2 << 4), A / B s8
  return (i8 ? ((2u << 4) | (1u << 7) | (1u << 10)) : ((1u << 4) | (1u << 7) | (1u << 10) | (1u << 15))) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(SK_BM >> 4) << 24);
}

template <bool I8>
__device__ __forceinline__ void skinny_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  if constexpr (I8) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

template <int RB, bool I8>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const SkinnyParams p) {
  using Cfg = SkinnyCfg<RB>;
  constexpr int BKE = I8 ? 128 : 64;                      // k elements per k-block (128 bytes of k for both types)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tmem_full = empty_bar + Cfg::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (p.N + SK_BM - 1) / SK_BM;
  const int num_kb = (p.K + BKE - 1) / BKE;
  const int items = nt * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tmap_w); prefetch_tmap(&tmap_x); }
  if (warp == 1) { tmem_alloc(tmem_holder, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < items && ok; t += gridDim.x) {
        const int split = t / nt, n_idx = t - split * nt;
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb_ = sa + SK_A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          if constexpr (I8) {
            // both maps are over 16-bit words (two int8 each): x = k / 2, boxes of 64 words = 128 bytes of k
            tma_load_2d(sa, &tmap_w, &full_bar[stage], kb * 64, n_idx * SK_BM);
            tma_load_2d(sb_, &tmap_x, &full_bar[stage], kb * 64, 0);
          } else {
            // W [K, N]: two boxes of 64 k x 64 columns (MN-major operand); X [rows, K]: one box of RB rows x 64 k
            tma_load_2d(sa, &tmap_w, &full_bar[stage], n_idx * SK_BM, kb * 64);
            tma_load_2d(sa + 8192, &tmap_w, &full_bar[stage], n_idx * SK_BM + 64, kb * 64);
            tma_load_2d(sb_, &tmap_x, &full_bar[stage], kb * 64, 0);
          }
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = skinny_idesc(I8, RB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < items && ok; t += gridDim.x, ++it) {
        const int split = t / nt;
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t sb_ = sa + SK_A_BYTES;
#pragma unroll
          for (int k = 0; k < 4; ++k) {               // four MMAs of 32 bytes of k each
            const uint64_t adesc = I8 ? make_smem_desc(sa + k * 32, 16, 1024)
                                      : make_smem_desc(sa + k * (16 * 128), 64 * 64 * 2, 1024);
            const uint64_t bdesc = make_smem_desc(sb_ + k * 32, 16, 1024);
            skinny_mma<I8>(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;                             // warps 2, 3, 4, 5 -> lane quarters 2, 3, 0, 1
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < items && ok; t += gridDim.x, ++it) {
      const int split = t / nt, n_idx = t - split * nt;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int col = n_idx * SK_BM + q * 32 + lane;    // this thread's output column
      const uint32_t taddr = tmem_base + acc * Cfg::ACC_STRIDE + (static_cast<uint32_t>(q * 32) << 16);
      float swc = 0.f;
      if constexpr (I8) swc = (col < p.N && p.splits == 1) ? p.sw[col] : 0.f;
#pragma unroll 1
      for (int c = 0; c < (RB + 31) / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (col < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = c * 32 + j;
            if (m < p.rows && m < RB) {
              if (p.splits == 1) {
                float v;
                if constexpr (I8) v = __fmul_rn(static_cast<float>(static_cast<int>(r[j])), __fmul_rn(p.sx[m], swc));
                else v = __uint_as_float(r[j]);
                if (p.R) v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.R)[static_cast<size_t>(m) * p.ldr + col]);
                static_cast<__nv_bfloat16*>(p.C)[static_cast<size_t>(m) * p.ldc + col] = __float2bfloat16_rn(v);
              } else {
                static_cast<uint32_t*>(p.C)[(static_cast<size_t>(split) * p.rows + m) * p.N + col] = r[j];
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// C[m, n] = bf16(sum over splits in split order (+ scales) + R[m, n])
template <bool I8>
__global__ void skinny_reduce_kernel(const void* __restrict__ part, int splits, int rows, int N,
                                     const float* __restrict__ sx, const float* __restrict__ sw,
                                     const __nv_bfloat16* __restrict__ R, int ldr, __nv_bfloat16* __restrict__ C,
                                     int ldc) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t mn = static_cast<size_t>(rows) * N;
  if (i >= mn) return;
  const int m = static_cast<int>(i / N), n = static_cast<int>(i - static_cast<size_t>(m) * N);
  float v;
  if constexpr (I8) {
    int acc = 0;
    for (int s = 0; s < splits; ++s) acc += static_cast<const int*>(part)[s * mn + i];
    v = __fmul_rn(static_cast<float>(acc), __fmul_rn(sx[m], sw[n]));
  } else {
    v = static_cast<const float*>(part)[i];
    for (int s = 1; s < splits; ++s) v += static_cast<const float*>(part)[s * mn + i];
  }
  if (R) v += __bfloat162float(R[static_cast<size_t>(m) * ldr + n]);
  C[static_cast<size_t>(m) * ldc + n] = __float2bfloat16_rn(v);
}

template <int RB, bool I8>
static int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, int grid,
                         cudaStream_t stream) {
  using Cfg = SkinnyCfg<RB>;
  auto kern = gemm_skinny_kernel<RB, I8>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr = true;
  }
  kern<<<grid, SK_THREADS, Cfg::SMEM_BYTES, stream>>>(tw, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

using namespace sb;

// C[rows, N] (bf16) = X . W (+ R), rows <= 64.
//   is_i8 == 0: X bf16 [rows, ldx], W bf16 [K, N] (row pitch ldw);
//   is_i8 == 1: X int8 [rows, ldx] with row scales sx, W int8 [N, K] (transposed codes, row pitch ldw, K % 16 == 0)
//               with column scales sw.
// Bases 16-byte aligned, pitches multiples of 16 bytes, N % 8 == 0. workspace: splits * rows * N 32-bit words, read
// only when the k range is split (splits <= 0 lets the launcher fill the GPU: about one work item per SM).
extern "C" int sb_gemm_skinny(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, const void* R, int ldr,
                              int rows, int N, int K, int is_i8, const float* sx, const float* sw, int splits,
                              void* workspace, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows <= 0 || rows > 64 || N <= 0 || K <= 0 || (N & 7) || !status) return SB_ERR_ARG;
  if (is_i8 && (!sx || !sw || (K & 15) || (ldx & 15) || (ldw & 15))) return SB_ERR_ARG;
  if (!is_i8 && ((ldx & 7) || (ldw & 7))) return SB_ERR_ALIGN;
  const int bke = is_i8 ? 128 : 64;
  const int num_kb = (K + bke - 1) / bke;
  const int nt = (N + SK_BM - 1) / SK_BM;
  if (splits <= 0) {
    splits = num_sms() / nt;                        // one work item per SM, no second round
    if (splits < 1) splits = 1;
    const int max_splits = num_kb / 4 > 0 ? num_kb / 4 : 1;      // at least four k-blocks per item
    if (splits > max_splits) splits = max_splits;
  }
  if (splits > num_kb) splits = num_kb;
  const int kbps = (num_kb + splits - 1) / splits;
  splits = (num_kb + kbps - 1) / kbps;
  if (splits > 1 && !workspace) return SB_ERR_ARG;
  const int rb = rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
  CUtensorMap tw, tx;
  int rc;
  if (is_i8) {
    rc = make_tmap_2d_bf16(&tw, W, static_cast<uint64_t>(K) / 2, N, static_cast<uint64_t>(ldw) / 2, 64, SK_BM);
    if (rc) return rc;
    rc = make_tmap_2d_bf16(&tx, X, static_cast<uint64_t>(K) / 2, rows, static_cast<uint64_t>(ldx) / 2, 64, rb);
  } else {
    rc = make_tmap_2d_bf16(&tw, W, N, K, ldw, 64, 64);
    if (rc) return rc;
    rc = make_tmap_2d_bf16(&tx, X, K, rows, ldx, 64, rb);
  }
  if (rc) return rc;
  SkinnyParams p;
  p.rows = rows; p.N = N; p.K = K; p.splits = splits; p.kb_per_split = kbps;
  p.C = splits > 1 ? workspace : C; p.ldc = ldc; p.R = R; p.ldr = ldr; p.sx = sx; p.sw = sw; p.status = status;
  const int items = nt * splits;
  const int grid = items < num_sms() ? items : num_sms();
#define SB_SKINNY(RB_)                                                              \
  rc = is_i8 ? launch_skinny<RB_, true>(tw, tx, p, grid, stream) : launch_skinny<RB_, false>(tw, tx, p, grid, stream)
  if (rb == 16) SB_SKINNY(16); else if (rb == 32) SB_SKINNY(32); else SB_SKINNY(64);
#undef SB_SKINNY
  if (rc) return rc;
  if (splits > 1) {
    const size_t mn = static_cast<size_t>(rows) * N;
    const unsigned blocks = static_cast<unsigned>((mn + 255) / 256);
    if (is_i8) skinny_reduce_kernel<true><<<blocks, 256, 0, stream>>>(workspace, splits, rows, N, sx, sw,
                                                                     static_cast<const __nv_bfloat16*>(R), ldr,
                                                                     static_cast<__nv_bfloat16*>(C), ldc);
    else skinny_reduce_kernel<false><<<blocks, 256, 0, stream>>>(workspace, splits, rows, N, nullptr, nullptr,
                                                                 static_cast<const __nv_bfloat16*>(R), ldr,
                                                                 static_cast<__nv_bfloat16*>(C), ldc);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  return 0;
}
