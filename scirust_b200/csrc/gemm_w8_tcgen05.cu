// int8 per-output-channel weight GEMM with the dequantisation fused into the operand path (W8A16):
//   C[M,N] = (A[M,K] (bf16) * Q[K,N] (int8)) * scale[n]  (+ R)
// Weights are stored as the reference's per-channel quantiser produces them for the x.W layout:
// int8 codes [K, N] and one fp32 scale per output column, W ~= Q * scale
// (scirust-core/src/quantization.rs:95-190; the shader INT8_GEMM applies the scales after the
// integer product the same way, scirust-gpu/src/kernels.rs:272).
//
// Pipeline per stage: TMA brings the bf16 A tile (128B-swizzled) and the raw int8 B tile
// [64 k x BN n]; four converter warps widen the codes to bf16 (exact: |q| <= 128) and write them
// in the MN-major 128B-swizzled layout tcgen05.mma reads; the MMA warp multiplies into TMEM; the
// epilogue multiplies each column by its scale. The weight bytes cross HBM once, as int8.
// Warps: 0 TMA, 1 MMA, 2-5 converters, 6-13 epilogue. K order is fixed; split-K partials are
// reduced in split order by w8_splitk_reduce_kernel (scale applied there).
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int num_sms();

constexpr int WBM = 128, WBK = 64, WBN = 256;
constexpr int W8_THREADS = 448;
constexpr int W8_STAGES = 3;
constexpr int W8_A_BYTES = WBM * WBK * 2;    // 16 KB
constexpr int W8_RAW_BYTES = WBK * WBN;      // 16 KB of int8
constexpr int W8_B_BYTES = WBN * WBK * 2;    // 32 KB of bf16
constexpr int W8_STAGE_BYTES = W8_A_BYTES + W8_RAW_BYTES + W8_B_BYTES;
constexpr int W8_SMEM_BYTES = W8_STAGES * W8_STAGE_BYTES + 1024 + 256;
constexpr int W8_TMEM_COLS = 2 * WBN;

struct W8Params {
  int M, N, K;
  int splits, kb_per_split;
  void* C; int ldc;          // bf16 [M, ldc], or fp32 [splits, M, N] partials
  const void* R; int ldr;
  const float* scale;
  int* status;
};

__global__ void __launch_bounds__(W8_THREADS, 1)
gemm_w8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_q,
               const W8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + W8_STAGES * W8_STAGE_BYTES);
  uint64_t* conv_bar = full_bar + W8_STAGES;
  uint64_t* empty_bar = conv_bar + W8_STAGES;
  uint64_t* tmem_full = empty_bar + W8_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = (p.M + WBM - 1) / WBM, nt = (p.N + WBN - 1) / WBN;
  const int num_kb = (p.K + WBK - 1) / WBK;
  const int tiles_total = mt * nt * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&conv_bar[s], 4);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 8); }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) { tmem_alloc(tmem_holder, W8_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x) {
        const int split = t / (mt * nt);
        const int rem = t - split * (mt * nt);
        const int n_idx = rem / mt, m_idx = rem - (rem / mt) * mt;
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * W8_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], W8_A_BYTES + W8_RAW_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * WBK, m_idx * WBM);
          tma_load_2d(sa + W8_A_BYTES, &tmap_q, &full_bar[stage], n_idx * WBN, kb * WBK);
          if (++stage == W8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(WBM, WBN, false, true);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x, ++it) {
        const int split = t / (mt * nt);
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        const int acc = it & 1;
        if (!mbar_wait(&tmem_empty[acc], ((it >> 1) & 1) ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * WBN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&conv_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * W8_STAGE_BYTES);
          const uint32_t sbf = sa + W8_A_BYTES + W8_RAW_BYTES;
#pragma unroll
          for (int k = 0; k < WBK / 16; ++k)
            umma_bf16_ss(d_tmem, make_smem_desc(sa + k * 32, 16, 1024),
                         make_smem_desc(sbf + k * (16 * 128), 64 * WBK * 2, 1024), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == W8_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else if (warp < 6) {
    // ---- converters: int8 [64 x 256] -> bf16 MN-major swizzled [4 chunks][64 k-rows][64 n] ----
    const int tid = threadIdx.x - 64;   // 0..127
    const int u = tid & 31;             // 8-column unit inside the 256-column tile
    const int r0 = tid >> 5;            // first k-row
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x) {
      const int split = t / (mt * nt);
      const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        // the A tile lands on the same barrier; waiting here also covers the raw B tile
        if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        const uint8_t* raw = smem + stage * W8_STAGE_BYTES + W8_A_BYTES;
        uint8_t* bt = smem + stage * W8_STAGE_BYTES + W8_A_BYTES + W8_RAW_BYTES;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int r = r0 + 4 * i;
          const uint2 q = *reinterpret_cast<const uint2*>(raw + r * WBN + u * 8);
          float f[8];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            f[b] = static_cast<float>(static_cast<int8_t>(q.x >> (8 * b)));
            f[4 + b] = static_cast<float>(static_cast<int8_t>(q.y >> (8 * b)));
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
          *reinterpret_cast<uint4*>(bt + (u >> 3) * (64 * WBK * 2) + r * 128 + (((u & 7) ^ (r & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv_bar[stage]);
        if (++stage == W8_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ---- epilogue ----
    const int q = warp & 3;
    const int half = (warp - 6) >> 2;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x, ++it) {
      const int split = t / (mt * nt);
      const int rem = t - split * (mt * nt);
      const int n_idx = rem / mt, m_idx = rem - (rem / mt) * mt;
      const int acc = it & 1;
      if (!mbar_wait(&tmem_full[acc], (it >> 1) & 1, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m_idx * WBM + q * 32 + lane;
      const uint32_t taddr_row = tmem_base + acc * WBN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = half * (WBN / 64); c < (half + 1) * (WBN / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_idx * WBN + c * 32;
        if (row < p.M && col0 < p.N) {
          if (p.splits == 1) {
            __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            const __nv_bfloat16* rrow =
                p.R ? static_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr + col0 : nullptr;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < p.N) {
                float f[8];
                const float4 s0 = *reinterpret_cast<const float4*>(p.scale + col0 + v * 8);
                const float4 s1 = *reinterpret_cast<const float4*>(p.scale + col0 + v * 8 + 4);
                const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]) * sc[j];
                if (rrow) {
                  const uint4 rv = *reinterpret_cast<const uint4*>(rrow + v * 8);
                  f[0] += bf16_lo(rv.x); f[1] += bf16_hi(rv.x); f[2] += bf16_lo(rv.y); f[3] += bf16_hi(rv.y);
                  f[4] += bf16_lo(rv.z); f[5] += bf16_hi(rv.z); f[6] += bf16_lo(rv.w); f[7] += bf16_hi(rv.w);
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(crow + v * 8) = o;
              }
            }
          } else {
            float* prow = static_cast<float*>(p.C) + (static_cast<size_t>(split) * p.M + row) * static_cast<size_t>(p.N) + col0;
#pragma unroll
            for (int v = 0; v < 8; ++v)
              if (col0 + v * 4 < p.N)
                *reinterpret_cast<uint4*>(prow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
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
  if (warp == 1) tmem_dealloc(tmem_base, W8_TMEM_COLS);
}

__global__ void w8_splitk_reduce_kernel(const float* __restrict__ part, int splits, size_t mn, int N,
                                        const float* __restrict__ scale, __nv_bfloat16* __restrict__ C, int ldc,
                                        const __nv_bfloat16* __restrict__ R, int ldr) {
  const size_t i4 = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i4 >= mn) return;
  float4 acc = *reinterpret_cast<const float4*>(part + i4);
  for (int s = 1; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(part + s * mn + i4);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const size_t row = i4 / N;
  const int col = static_cast<int>(i4 - row * N);
  const float4 sc = *reinterpret_cast<const float4*>(scale + col);
  acc.x *= sc.x; acc.y *= sc.y; acc.z *= sc.z; acc.w *= sc.w;
  if (R) {
    const uint2 rv = *reinterpret_cast<const uint2*>(R + row * ldr + col);
    acc.x += bf16_lo(rv.x); acc.y += bf16_hi(rv.x); acc.z += bf16_lo(rv.y); acc.w += bf16_hi(rv.y);
  }
  uint2 o;
  o.x = pack_bf16x2(acc.x, acc.y);
  o.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(C + row * ldc + col) = o;
}

typedef CUresult (*EncodeTiledFn8)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld_bytes,
                           uint32_t box_inner, uint32_t box_outer) {
  thread_local bool context_bound = false;      // the driver call below wants a context current on this thread
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  static EncodeTiledFn8 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return SB_ERR_DRIVER;
    fn = reinterpret_cast<EncodeTiledFn8>(ptr);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld_bytes & 15)) return SB_ERR_ALIGN;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SB_ERR_DRIVER;
}

}  // namespace sb

using namespace sb;

// C[M,N] = (A[M,K] * Q[K,N]) * scale[n] (+ R). Q int8 with row pitch ldq bytes (multiple of 16), N a
// multiple of 16. splits > 1 needs `workspace` of splits*M*N floats.
extern "C" int sb_gemm_w8(const void* A, const void* Q, const float* scale, void* C, const void* R, int M, int N,
                          int K, int lda, int ldq, int ldc, int ldr, int splits, void* workspace, int* status,
                          void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || (N & 15) || (ldc & 7) || (ldq & 15) || (R && (ldr & 7))) return SB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(scale) & 15)) return SB_ERR_ALIGN;
  const int num_kb = (K + WBK - 1) / WBK;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  const int kps = (num_kb + splits - 1) / splits;
  splits = (num_kb + kps - 1) / kps;
  if (splits > 1 && !workspace) return SB_ERR_ARG;
  CUtensorMap ta, tq;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, WBK, WBM);
  if (rc) return rc;
  rc = make_tmap_2d_u8(&tq, Q, N, K, ldq, WBN, WBK);
  if (rc) return rc;
  W8Params p;
  p.M = M; p.N = N; p.K = K; p.splits = splits; p.kb_per_split = kps;
  p.C = splits > 1 ? workspace : C;
  p.ldc = ldc;
  p.R = splits > 1 ? nullptr : R;
  p.ldr = ldr;
  p.scale = scale;
  p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_w8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W8_SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  const int tiles = ((M + WBM - 1) / WBM) * ((N + WBN - 1) / WBN) * splits;
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_w8_kernel<<<grid, W8_THREADS, W8_SMEM_BYTES, stream>>>(ta, tq, p);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  if (splits > 1) {
    const size_t mn = static_cast<size_t>(M) * N;
    w8_splitk_reduce_kernel<<<static_cast<unsigned>((mn / 4 + 255) / 256), 256, 0, stream>>>(
        static_cast<const float*>(workspace), splits, mn, N, scale, static_cast<__nv_bfloat16*>(C), ldc,
        static_cast<const __nv_bfloat16*>(R), ldr);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  return 0;
}
