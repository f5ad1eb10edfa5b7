// Timing probe for tcgen05.mma (kind::f16, bf16 operands from shared memory, cta_group::1): one
// thread of one CTA issues a long series of instructions of one shape into the same accumulator and
// the cycles per instruction are read from the SM clock. It answers how the cost of an instruction
// depends on M and N, which decides tile shapes where one dimension is small (attention with head
// dimension 64: N = 64 in P V, dK and dV).
#include "sm100_ptx.cuh"
#include "api.h"

namespace sb {

template <bool B_MN>
__global__ void __launch_bounds__(128, 1)
umma_probe_kernel(int M, int N, int iters, long long* out_cycles, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                  // 128 rows x 64 bf16, 128-byte swizzled K-major
  uint8_t* sB = smem + 16384;          // 256 rows x 64 bf16 (K-major) or 64 k-rows x 256 (MN-major: 4 chunks of 64)
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 16384 + 32768);
  uint32_t* holder = reinterpret_cast<uint32_t*>(bar + 1);
  for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);   // bf16 ones
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc(holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(holder);
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_bf16(M, N, false, B_MN);
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint64_t adesc = make_smem_desc(a0 + k * 32, 16, 1024);
        const uint64_t bdesc = B_MN ? make_smem_desc(b0 + k * (16 * 128), 64 * 128, 1024)
                                    : make_smem_desc(b0 + k * 32, 16, 1024);
        umma_bf16_ss(tmem_base, adesc, bdesc, idesc, 1u);
      }
    }
    const long long t_issue = clock64();
    umma_commit(bar);
    const bool ok = mbar_wait(bar, 0, status, ST_TIMEOUT_TMEM_FULL);
    const long long t1 = clock64();
    out_cycles[0] = ok ? (t1 - t0) : -1;
    out_cycles[1] = t_issue - t0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem_base, 512);
}

}  // namespace sb

// out_cycles[0] = cycles from the first issue to completion of 4 * iters instructions (-1 on a
// wait that ran out), out_cycles[1] = cycles spent issuing. M in {64, 128}, N a multiple of 16 up
// to 256; b_mn selects an MN-major B operand (the layout of a [k][n] row-major tile such as V).
extern "C" int sb_umma_probe(int M, int N, int b_mn, int iters, long long* out_cycles, int* status, void* stream_) {
  if ((M != 64 && M != 128) || N < 16 || N > 256 || (N % 16) || iters <= 0 || iters > 100000) return SB_ERR_ARG;
  const int smem_bytes = 16384 + 32768 + 64 + 1024;
  auto k0 = sb::umma_probe_kernel<false>;
  auto k1 = sb::umma_probe_kernel<true>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess ||
        cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess)
      return SB_ERR_LAUNCH;
    attr_set = true;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (b_mn) k1<<<1, 128, smem_bytes, stream>>>(M, N, iters, out_cycles, status);
  else k0<<<1, 128, smem_bytes, stream>>>(M, N, iters, out_cycles, status);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
