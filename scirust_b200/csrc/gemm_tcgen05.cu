// bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[M,N] = op(A) * op(B)   with fp32 accumulation in tensor memory.
//
// Replaces the three cuBLASLt forms the reference drives (A*B, A*B^T, A^T*B:
// scirust-cuda/src/chain.rs:1037-1083, 1177-1215, 1228-1266) and folds the
// reference's separate residual `add_kernel` (chain.rs:40) into the epilogue.
//
// Operand forms are expressed by the *major-ness* of each operand in memory:
//   A "K-major":  A stored [M, K] row-major (K contiguous)
//   A "MN-major": A stored [K, M] row-major (M contiguous)      (i.e. A^T * ...)
//   B "K-major":  B stored [N, K] row-major (K contiguous)      (i.e. ... * B^T)
//   B "MN-major": B stored [K, N] row-major (N contiguous)
// so  X*W      (W [in,out])  = A K-major,  B MN-major
//     dY*W^T                 = A K-major,  B K-major
//     X^T*dY   (weight grad) = A MN-major, B MN-major
//
// Kernel shape: persistent, one CTA per SM, 10 warps:
//   warp 0   TMA producer (one elected lane)
//   warp 1   MMA issuer (one elected lane); owns the TMEM allocation
//   warp 2-9 epilogue: a warp may touch the 32 TMEM lanes of quarter (warp_id % 4); the two
//            warps of a quarter split the tile's columns
// Two fp32 accumulators (2 x BN columns of TMEM) let the epilogue of tile i overlap the
// main loop of tile i+1. K is walked in a fixed order, so results are bitwise
// repeatable; split-K writes fp32 partials that a second kernel adds in split order.
#include <stdio.h>
#include "sm100_ptx.cuh"
#include "api.h"
#include "gemm_sched.cuh"

namespace sb {

constexpr int BM = 128;
constexpr int BK = 64;       // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;  // 512 or 256: both powers of two
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct GemmParams {
  int M, N, K;
  int splits;          // explicit split-K factor (1 = none)
  int kb_per_split;    // k-blocks per split
  void* C;             // bf16 [M, ldc] when splits == 1; fp32 [splits, M, N] partials otherwise
  int ldc;
  const void* R;       // optional bf16 residual [M, ldr] added in the epilogue (splits == 1)
  int ldr;
  int* status;
  BalancedSched sched;   // balanced schedule (splits == 1 only); see gemm_sched.cuh
  float* partials;       // scratch slots of the balanced schedule: dense fp32 [BM, BN] blocks
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tmem_full = empty_bar + Cfg::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int mt = (p.M + BM - 1) / BM;
  const int nt = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_mn = mt * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
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
      SegIter iter(p.sched, blockIdx.x, gridDim.x, tiles_mn, num_kb, p.splits, p.kb_per_split);
      Seg sg;
      while (ok && iter.next(sg)) {
        const int n_idx = sg.tile / mt;
        const int m_idx = sg.tile - n_idx * mt;
        const int kb0 = sg.kb0, kb1 = sg.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb_ = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m_idx * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (64 * BK * 2), &tmap_a, &full_bar[stage], m_idx * BM + c * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb_, &tmap_b, &full_bar[stage], kb * BK, n_idx * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb_ + c * (64 * BK * 2), &tmap_b, &full_bar[stage], n_idx * BN + c * 64, kb * BK);
          }
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      SegIter iter(p.sched, blockIdx.x, gridDim.x, tiles_mn, num_kb, p.splits, p.kb_per_split);
      Seg sg;
      for (; ok && iter.next(sg); ++it) {
        const int kb0 = sg.kb0, kb1 = sg.kb1;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t sb_ = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb_ + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc(sb_ + k * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    bool ok = true;
    int it = 0;
    SegIter iter(p.sched, blockIdx.x, gridDim.x, tiles_mn, num_kb, p.splits, p.kb_per_split);
    Seg sg;
    for (; ok && iter.next(sg); ++it) {
      const int split = sg.split;
      const int n_idx = sg.tile / mt;
      const int m_idx = sg.tile - n_idx * mt;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m_idx * BM + q * 32 + lane;
      const uint32_t taddr_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_idx * BN + c * 32;
        if (sg.slot >= 0) {
          // part of a tile of the balanced schedule: dense fp32 block, finished by the fix-up kernel
          float* prow = p.partials + (static_cast<size_t>(sg.slot) * BM + (q * 32 + lane)) * BN + c * 32;
#pragma unroll
          for (int v = 0; v < 8; ++v)
            *reinterpret_cast<uint4*>(prow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        } else if (row < p.M && col0 < p.N) {
          if (p.splits == 1) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            const __nv_bfloat16* rrow =
                p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr + col0
                    : nullptr;
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
          } else {
            float* prow = reinterpret_cast<float*>(p.C) +
                          (static_cast<size_t>(split) * p.M + row) * static_cast<size_t>(p.N) + col0;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (col0 + v * 4 < p.N) {  // N % 8 == 0
                *reinterpret_cast<uint4*>(prow + v * 4) =
                    make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
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

  // Teardown: every role loop above is bounded, so all threads arrive here.
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// Adds split-K partials in split order 0..S-1 (fixed order => bitwise repeatable),
// optionally adds a bf16 residual, rounds to bf16.
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, size_t mn, int N,
                                     __nv_bfloat16* __restrict__ C, int ldc, const __nv_bfloat16* __restrict__ R,
                                     int ldr) {
  const size_t i4 = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i4 >= mn) return;
  float4 acc = *reinterpret_cast<const float4*>(part + i4);
  for (int s = 1; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(part + s * mn + i4);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const size_t row = i4 / N;
  const int col = static_cast<int>(i4 - row * N);
  if (R) {
    const uint2 rv = *reinterpret_cast<const uint2*>(R + row * ldr + col);
    acc.x += bf16_lo(rv.x); acc.y += bf16_hi(rv.x);
    acc.z += bf16_lo(rv.y); acc.w += bf16_hi(rv.y);
  }
  uint2 o;
  o.x = pack_bf16x2(acc.x, acc.y);
  o.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(C + row * ldc + col) = o;
}

// ------------------------------ host side ------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  // cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread. A thread that has
  // only ever used device 0 through a framework that skips cudaSetDevice when "the device is already 0" (an autograd
  // worker whose first native call is a tensor-map encode) has none: bind the primary context once per thread.
  thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      fprintf(stderr, "scirust_b200: cuTensorMapEncodeTiled could not be resolved\n");
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map with 128B swizzle. `inner` elements are contiguous; `ld` is
// the row pitch in elements. Returns 0 on success.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return SB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return SB_ERR_ALIGN;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "scirust_b200: tensor map refused (driver code %d): base %p, dims %llu x %llu, pitch %llu B, box %u x %u\n",
            static_cast<int>(r), base, static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
            static_cast<unsigned long long>(ld * 2), box_inner, box_outer);
  return r == CUDA_SUCCESS ? 0 : SB_ERR_DRIVER;
}

// 3-D bf16 tensor map with 128B swizzle: dims (d0 contiguous, d1, d2), pitches in elements; the box is
// box0 x box1 x 1. Out-of-range parts of a box are zero on loads and dropped on stores.
int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t box0, uint32_t box1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return SB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((pitch1 * 2) & 15) || ((pitch2 * 2) & 15)) return SB_ERR_ALIGN;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1 * 2, pitch2 * 2};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SB_ERR_DRIVER;
}

// 2-D tensor map over 16-bit words without swizzle (row-major copy of a box into shared memory).
// Used by the weight-streaming kernels: `inner` 2-byte words are contiguous, `pitch_bytes` is the row
// pitch. Out-of-range parts of a box are filled with zeros.
int make_tmap_2d_u16_plain(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                           uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return SB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15)) return SB_ERR_ALIGN;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SB_ERR_DRIVER;
}

static int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

using namespace sb;

// C[M,N] (bf16, pitch ldc) = op(A) op(B) (+ R).  a_mn / b_mn select the operand
// major-ness described at the top of this file; lda/ldb are row pitches (elements)
// of the matrices as stored. `splits` > 1 is explicit split-K and needs `workspace` of
// splits*M*N floats. `splits` == 0 selects the balanced schedule (whole waves of tiles one per
// CTA, the k-blocks of the last partial wave dealt out evenly over all SMs); it needs `workspace`
// of sb_gemm_balanced_workspace_floats() floats and falls back to one tile per CTA without it.
// bn: 0 = choose, else 128 or 256.
extern "C" size_t sb_gemm_balanced_workspace_floats() { return static_cast<size_t>(num_sms()) * 3 * BM * 256; }

extern "C" int sb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda,
                            int ldb, int ldc, int ldr, int a_mn, int b_mn, int splits, void* workspace, int bn,
                            int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return SB_ERR_ARG;
  if ((N & 7) || (ldc & 7) || (R && (ldr & 7))) return SB_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(C) & 15) return SB_ERR_ALIGN;
  if (R && (reinterpret_cast<uintptr_t>(R) & 15)) return SB_ERR_ALIGN;
  const int num_kb = (K + BK - 1) / BK;
  const bool balanced = splits == 0 && workspace != nullptr;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  int kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per_split - 1) / kb_per_split;  // no empty split
  if (splits > 1 && !workspace) return SB_ERR_ARG;
  if (bn == 0) bn = (N <= 128) ? 128 : 256;
  if (bn != 128 && bn != 256) return SB_ERR_ARG;

  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  else rc = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, bn);
  else rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.splits = splits;
  p.kb_per_split = kb_per_split;
  p.C = splits > 1 ? workspace : C;
  p.ldc = ldc;
  p.R = splits > 1 ? nullptr : R;
  p.ldr = ldr;
  p.status = status;
  p.partials = nullptr;
  const int mt = (M + BM - 1) / BM, nt = (N + bn - 1) / bn;
  const int tiles = mt * nt * splits;
  int grid = tiles < num_sms() ? tiles : num_sms();
  bool fixup = false;
  if (balanced && plan_balanced(tiles, num_kb, num_sms(), &p.sched, &fixup)) {
    p.partials = static_cast<float*>(workspace);
    grid = p.sched.dp_tiles > 0 ? num_sms() : p.sched.sk_workers;
  } else {
    p.sched.dp_tiles = p.sched.sk_tiles = p.sched.sk_workers = p.sched.sk_slots = 0;
  }

#define SB_DISPATCH(BN_)                                                                   \
  do {                                                                                     \
    if (!a_mn && !b_mn) rc = launch_gemm<BN_, false, false>(ta, tb, p, grid, stream);      \
    else if (!a_mn && b_mn) rc = launch_gemm<BN_, false, true>(ta, tb, p, grid, stream);   \
    else if (a_mn && !b_mn) rc = launch_gemm<BN_, true, false>(ta, tb, p, grid, stream);   \
    else rc = launch_gemm<BN_, true, true>(ta, tb, p, grid, stream);                       \
  } while (0)
  if (bn == 256) SB_DISPATCH(256); else SB_DISPATCH(128);
#undef SB_DISPATCH
  if (rc) return rc;

  if (fixup) {
    dim3 fg(p.sched.sk_tiles, BM * bn / (256 * 4));
    __nv_bfloat16* c = static_cast<__nv_bfloat16*>(C);
    const __nv_bfloat16* r = static_cast<const __nv_bfloat16*>(R);
    if (bn == 256) balanced_fixup_kernel<BM, 256><<<fg, 256, 0, stream>>>(p.sched, p.partials, c, ldc, r, ldr, M, N, mt, num_kb);
    else balanced_fixup_kernel<BM, 128><<<fg, 256, 0, stream>>>(p.sched, p.partials, c, ldc, r, ldr, M, N, mt, num_kb);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  if (splits > 1) {
    const size_t mn = static_cast<size_t>(M) * N;
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((mn / 4 + threads - 1) / threads);
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(static_cast<const float*>(workspace), splits, mn, N,
                                                         static_cast<__nv_bfloat16*>(C), ldc,
                                                         static_cast<const __nv_bfloat16*>(R), ldr);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  return 0;
}
