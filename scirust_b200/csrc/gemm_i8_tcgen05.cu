// W8A8 GEMM on the integer tensor cores: C[M,N] = (Xq[M,K] (int8) . Wq[N,K]^T (int8)) * sx[m] * sw[n] (+ R)
//
// The reference's quantised linear layer quantises the activations per row on the fly (scale = max|x| / 127, round
// half away from zero), multiplies int8 x int8 into int32 and rescales once by the product of the row and column
// scales (scirust-core/src/quantization.rs:150-190, `quantized_linear_forward`). This is that arithmetic, exactly
// (integer accumulation has no rounding, so the result does not depend on tile shapes, k order or split-K), on
// tcgen05.mma.kind::i8: the weight bytes cross HBM once as int8 and go from TMA straight into the MMA, with no
// conversion stage in between, so batched decoding (M of 16 to a few hundred rows) streams weights at the copy rate.
//
// Both operands are K-major ([rows, K], K contiguous): Xq as the row quantiser writes it, the weights as the
// transposed int8 copy kept for this kernel. A 128-byte swizzle row holds 128 k, an MMA consumes 32 of them, so the
// shared-memory descriptors advance by 32 bytes per MMA exactly as in the bf16 K-major kernel.
// Warps: 0 TMA, 1 MMA, 2-9 epilogue (int32 -> fp32, scales, residual, bf16). Split-K partials are int32 and are added
// by i8_splitk_reduce_kernel, which applies the scales.
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
int num_sms();

constexpr int I8_BM = 128, I8_BN = 256, I8_BK = 128, I8_UMMA_K = 32;
constexpr int I8_THREADS = 320;
constexpr int I8_STAGES = 4;
constexpr int I8_A_BYTES = I8_BM * I8_BK;      // 16 KB
constexpr int I8_B_BYTES = I8_BN * I8_BK;      // 32 KB
constexpr int I8_STAGE_BYTES = I8_A_BYTES + I8_B_BYTES;
constexpr int I8_SMEM_BYTES = I8_STAGES * I8_STAGE_BYTES + 1024 + 256;
constexpr int I8_TMEM_COLS = 2 * I8_BN;

// Instruction descriptor of tcgen05.mma.kind::i8: [4,6) D format 2 = s32, [7,10) A format 1 = signed 8-bit,
// [10,13) B format 1 = signed 8-bit, both operands K-major, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct I8Params {
  int M, N, K;
  int splits, kb_per_split;
  void* C; int ldc;            // bf16 [M, ldc], or int32 [splits, M, N] partials
  const void* R; int ldr;
  const float* sx;             // [M] activation row scales
  const float* sw;             // [N] weight column scales
  int* status;
};

__global__ void __launch_bounds__(I8_THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const I8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + I8_STAGES * I8_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + I8_STAGES;
  uint64_t* tmem_full = empty_bar + I8_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = (p.M + I8_BM - 1) / I8_BM, nt = (p.N + I8_BN - 1) / I8_BN;
  const int num_kb = (p.K + I8_BK - 1) / I8_BK;
  const int tiles_total = mt * nt * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < I8_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 8); }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tmap_a); prefetch_tmap(&tmap_b); }
  if (warp == 1) { tmem_alloc(tmem_holder, I8_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  // work item t: split = t / (mt * nt), tile = t % (mt * nt), n index major so that CTAs next to one another share A
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x) {
        const int split = t / (mt * nt), tile = t - split * (mt * nt);
        const int n_idx = tile / mt, m_idx = tile - n_idx * mt;
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = tiles + stage * I8_STAGE_BYTES;
          uint8_t* sb_ = sa + I8_A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], I8_STAGE_BYTES);
          // the maps are over 16-bit words (two int8 each): x = k / 2, a box is 64 words = 128 bytes wide;
          // rows past M / N and k past K arrive as zeros
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * (I8_BK / 2), m_idx * I8_BM);
          tma_load_2d(sb_, &tmap_b, &full_bar[stage], kb * (I8_BK / 2), n_idx * I8_BN);
          if (++stage == I8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8(I8_BM, I8_BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x, ++it) {
        const int split = t / (mt * nt);
        const int kb0 = split * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * I8_BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * I8_STAGE_BYTES);
          const uint32_t sb_ = sa + I8_A_BYTES;
#pragma unroll
          for (int k = 0; k < I8_BK / I8_UMMA_K; ++k) {
            const uint64_t adesc = make_smem_desc(sa + k * I8_UMMA_K, 16, 1024);
            const uint64_t bdesc = make_smem_desc(sb_ + k * I8_UMMA_K, 16, 1024);
            umma_i8_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == I8_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < tiles_total && ok; t += gridDim.x, ++it) {
      const int split = t / (mt * nt), tile = t - split * (mt * nt);
      const int n_idx = tile / mt, m_idx = tile - n_idx * mt;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m_idx * I8_BM + q * 32 + lane;
      const uint32_t taddr_row = tmem_base + acc * I8_BN + (static_cast<uint32_t>(q * 32) << 16);
      const float sxr = (row < p.M && p.splits == 1) ? p.sx[row] : 0.f;
#pragma unroll 1
      for (int c = half * (I8_BN / 64); c < (half + 1) * (I8_BN / 64); ++c) {
        const int col0 = n_idx * I8_BN + c * 32;
        if (m_idx * I8_BM + q * 32 >= p.M || col0 >= p.N) continue;      // whole warp: nothing live in this chunk
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c * 32, r);
        tmem_ld_wait();
        if (row >= p.M) continue;
        if (p.splits == 1) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
          const __nv_bfloat16* rrow =
              p.R ? reinterpret_cast<const __nv_bfloat16*>(p.R) + static_cast<size_t>(row) * p.ldr + col0 : nullptr;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p.N) {   // N % 8 == 0 is enforced on the host
              const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.sw + col0 + v * 8));
              const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.sw + col0 + v * 8 + 4));
              const float sw8[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                f[j] = __fmul_rn(static_cast<float>(static_cast<int>(r[v * 8 + j])), __fmul_rn(sxr, sw8[j]));   // never an FMA with the residual
              if (rrow) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + v * 8);
                f[0] += bf16_lo(rv.x); f[1] += bf16_hi(rv.x); f[2] += bf16_lo(rv.y); f[3] += bf16_hi(rv.y);
                f[4] += bf16_lo(rv.z); f[5] += bf16_hi(rv.z); f[6] += bf16_lo(rv.w); f[7] += bf16_hi(rv.w);
              }
              *reinterpret_cast<uint4*>(crow + v * 8) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                                   pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
            }
          }
        } else {
          int* prow = reinterpret_cast<int*>(p.C) + (static_cast<size_t>(split) * p.M + row) * static_cast<size_t>(p.N) + col0;
#pragma unroll
          for (int v = 0; v < 8; ++v)
            if (col0 + v * 4 < p.N)
              *reinterpret_cast<uint4*>(prow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
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
  if (warp == 1) tmem_dealloc(tmem_base, I8_TMEM_COLS);
}

// out[m, n] = bf16((sum over splits of part[s, m, n]) * sx[m] * sw[n] + R[m, n]); integer sums: any order, same bits
__global__ void i8_splitk_reduce_kernel(const int* __restrict__ part, int splits, int M, int N,
                                        const float* __restrict__ sx, const float* __restrict__ sw,
                                        const __nv_bfloat16* __restrict__ R, int ldr, __nv_bfloat16* __restrict__ C,
                                        int ldc) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<size_t>(M) * N) return;
  const int m = static_cast<int>(i / N), n = static_cast<int>(i - static_cast<size_t>(m) * N);
  int acc = 0;
  for (int s = 0; s < splits; ++s) acc += part[(static_cast<size_t>(s) * M + m) * N + n];
  float v = __fmul_rn(static_cast<float>(acc), __fmul_rn(sx[m], sw[n]));
  if (R) v += __bfloat162float(R[static_cast<size_t>(m) * ldr + n]);
  C[static_cast<size_t>(m) * ldc + n] = __float2bfloat16_rn(v);
}

// One warp per row: scale = max|x| / 127 (1 for a zero row), q = clamp(round half away from zero (x / scale)).
__global__ void quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int8_t* __restrict__ q, int ldq,
                                     float* __restrict__ sx, int M, int K) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  float amax = 0.f;
  for (int k = lane; k < K; k += 32) amax = fmaxf(amax, fabsf(__bfloat162float(xr[k])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax == 0.f ? 1.f : amax / 127.f;
  if (lane == 0) sx[row] = s;
  int8_t* qr = q + static_cast<size_t>(row) * ldq;
  for (int k = lane; k < K; k += 32) {
    const float v = __fdiv_rn(__bfloat162float(xr[k]), s);
    float r = v >= 0.f ? floorf(v + 0.5f) : ceilf(v - 0.5f);
    r = fminf(fmaxf(r, -128.f), 127.f);
    qr[k] = static_cast<int8_t>(r);
  }
}

// The same quantiser, one CTA per row, eight elements (16 bytes) per thread and step: the row is read once from
// memory (the second pass hits L1 / L2), the maximum is combined through shared memory.
__global__ void __launch_bounds__(256)
quantize_rows_vec8_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int8_t* __restrict__ q, int ldq,
                          float* __restrict__ sx, int K) {
  __shared__ float s_max[8];
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx);
  const int n8 = K >> 3;
  float amax = 0.f;
  for (int i = threadIdx.x; i < n8; i += 256) {
    const uint4 v = xr[i];
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf16_lo(v.x)), fabsf(bf16_hi(v.x))), fmaxf(fabsf(bf16_lo(v.y)), fabsf(bf16_hi(v.y)))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf16_lo(v.z)), fabsf(bf16_hi(v.z))), fmaxf(fabsf(bf16_lo(v.w)), fabsf(bf16_hi(v.w)))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) s_max[warp] = amax;
  __syncthreads();
  amax = s_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_max[w]);
  const float s = amax == 0.f ? 1.f : amax / 127.f;
  if (threadIdx.x == 0) sx[row] = s;
  uint2* qr = reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * ldq);
  for (int i = threadIdx.x; i < n8; i += 256) {
    const uint4 v = xr[i];
    const float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                        bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = __fdiv_rn(f[j], s);
      float r = t >= 0.f ? floorf(t + 0.5f) : ceilf(t - 0.5f);
      r = fminf(fmaxf(r, -128.f), 127.f);
      w[j >> 2] |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xffu) << (8 * (j & 3));
    }
    qr[i] = make_uint2(w[0], w[1]);
  }
}

}  // namespace sb

using namespace sb;

#define STREAM static_cast<cudaStream_t>(stream)

// xq [M, ldq] int8 (ldq >= K, a multiple of 16), sx [M] from the bf16 activations x [M, ldx].
extern "C" int sb_quantize_rows(const void* x, int ldx, void* xq, int ldq, float* sx, int M, int K, void* stream) {
  if (M <= 0 || K <= 0 || ldq < K) return SB_ERR_ARG;
  if ((K & 7) == 0 && (ldx & 7) == 0 && (ldq & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(xq) & 7) == 0) {
    quantize_rows_vec8_kernel<<<M, 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                     static_cast<int8_t*>(xq), ldq, sx, K);
    return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
  }
  quantize_rows_kernel<<<(M + 7) / 8, 256, 0, STREAM>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                        static_cast<int8_t*>(xq), ldq, sx, M, K);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// C[M, N] (bf16) = (xq . wq_t^T) * sx[m] * sw[n] (+ R). xq [M, ldq] int8, wq_t [N, ldw] int8 (both K contiguous; bases
// 16-byte aligned, pitches multiples of 16), K a multiple of 16, N a multiple of 8. workspace: splits * M * N int32
// (only read when splits > 1).
extern "C" int sb_gemm_i8(const void* xq, int ldq, const float* sx, const void* wq_t, int ldw, const float* sw, void* C,
                          int ldc, const void* R, int ldr, int M, int N, int K, int splits, void* workspace,
                          int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 15) || (ldq & 15) || (ldw & 15) || !sx || !sw || !status)
    return SB_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(sw) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) || ((ldc * 2) & 15)) return SB_ERR_ALIGN;
  if (R && ((reinterpret_cast<uintptr_t>(R) & 15) || ((ldr * 2) & 15))) return SB_ERR_ALIGN;
  const int num_kb = (K + I8_BK - 1) / I8_BK;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  int kbps = (num_kb + splits - 1) / splits;
  splits = (num_kb + kbps - 1) / kbps;
  if (splits > 1 && !workspace) return SB_ERR_ARG;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, xq, static_cast<uint64_t>(K) / 2, M, static_cast<uint64_t>(ldq) / 2, 64, I8_BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, wq_t, static_cast<uint64_t>(K) / 2, N, static_cast<uint64_t>(ldw) / 2, 64, I8_BN);
  if (rc) return rc;
  I8Params p;
  p.M = M; p.N = N; p.K = K; p.splits = splits; p.kb_per_split = kbps;
  p.C = splits == 1 ? C : workspace; p.ldc = ldc; p.R = R; p.ldr = ldr; p.sx = sx; p.sw = sw; p.status = status;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, I8_SMEM_BYTES) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr = true;
  }
  const int mt = (M + I8_BM - 1) / I8_BM, nt = (N + I8_BN - 1) / I8_BN;
  const int total = mt * nt * splits;
  const int grid = total < num_sms() ? total : num_sms();
  gemm_i8_kernel<<<grid, I8_THREADS, I8_SMEM_BYTES, STREAM>>>(ta, tb, p);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  if (splits > 1) {
    const size_t n = static_cast<size_t>(M) * N;
    i8_splitk_reduce_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, STREAM>>>(
        static_cast<const int*>(workspace), splits, M, N, sx, sw, static_cast<const __nv_bfloat16*>(R), ldr,
        static_cast<__nv_bfloat16*>(C), ldc);
    if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  }
  return 0;
}
