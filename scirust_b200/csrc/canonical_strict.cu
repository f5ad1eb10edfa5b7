// Canonical elementwise / permute kernels: the small fixed operator set whose results must agree
// bit for bit with the CPU interpreter (scirust-gpu/src/cuda_reference.rs:498-520 for the operator
// list and arities, :684-790 for the per-operator rules, :792-890 for permute). Compiled with
// contraction, flush-to-zero and approximate division off; arithmetic goes through the
// round-to-nearest intrinsics so that no flag can change it. Exp and Log are not provided: no
// implementation of them is bit-reproducible across targets, and the reference refuses them too.
//
//   relu   : NaN and strictly positive inputs pass through as raw words (NaN payloads survive),
//            everything else, -0.0 included, becomes +0.0
//   scale  : x * factor, factor given by its bit pattern
//   add, sub, mul, div : IEEE-754 binary32, round to nearest even
//   copy   : 32-bit words
//   permute: out[i] = in[sum_k idx_k(i) * in_stride[perm[k]]], words, rank <= 8
// Grid-stride loops, 256 threads per block.
#include <cuda_runtime.h>
#include <stdint.h>
#include "api.h"

namespace sb {

enum : int { CANON_RELU = 0, CANON_SCALE = 1, CANON_ADD = 2, CANON_SUB = 3, CANON_MUL = 4, CANON_DIV = 5, CANON_COPY = 6 };

__global__ void __launch_bounds__(256)
canon_elementwise_kernel(int op, const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, uint32_t* __restrict__ out,
                         long long n, uint32_t factor_bits) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint32_t xa = a[i];
    uint32_t r;
    switch (op) {
      case CANON_RELU: {
        const bool is_nan = ((xa & 0x7f800000u) == 0x7f800000u) && ((xa & 0x007fffffu) != 0u);
        r = (is_nan || __uint_as_float(xa) > 0.0f) ? xa : 0u;
        break;
      }
      case CANON_SCALE: r = __float_as_uint(__fmul_rn(__uint_as_float(xa), __uint_as_float(factor_bits))); break;
      case CANON_ADD: r = __float_as_uint(__fadd_rn(__uint_as_float(xa), __uint_as_float(b[i]))); break;
      case CANON_SUB: r = __float_as_uint(__fsub_rn(__uint_as_float(xa), __uint_as_float(b[i]))); break;
      case CANON_MUL: r = __float_as_uint(__fmul_rn(__uint_as_float(xa), __uint_as_float(b[i]))); break;
      case CANON_DIV: r = __float_as_uint(__fdiv_rn(__uint_as_float(xa), __uint_as_float(b[i]))); break;
      default: r = xa; break;
    }
    out[i] = r;
  }
}

struct PermuteArgs {
  int rank;
  long long out_shape[8];
  long long in_stride[8];   // stride of the input axis that feeds output axis k
};

__global__ void __launch_bounds__(256)
canon_permute_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, long long n, PermuteArgs pa) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    long long rem = i, src = 0;
    for (int k = pa.rank - 1; k >= 0; --k) {
      const long long idx = rem % pa.out_shape[k];
      rem /= pa.out_shape[k];
      src += idx * pa.in_stride[k];
    }
    out[i] = in[src];
  }
}

static int grid_for(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return g < 1 ? 1 : static_cast<int>(g);
}

}  // namespace sb

using namespace sb;

// op: 0 relu, 1 scale, 2 add, 3 sub, 4 mul, 5 div, 6 copy. b is ignored by the one-operand operators.
extern "C" int sb_canon_elementwise(int op, const void* a, const void* b, void* out, long long n, uint32_t factor_bits,
                                    void* stream_) {
  if (op < CANON_RELU || op > CANON_COPY || n < 0 || !a || !out) return SB_ERR_ARG;
  if (op >= CANON_ADD && op <= CANON_DIV && !b) return SB_ERR_ARG;
  if (n == 0) return 0;
  canon_elementwise_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      op, static_cast<const uint32_t*>(a), static_cast<const uint32_t*>(b), static_cast<uint32_t*>(out), n, factor_bits);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// in_shape[rank] is the shape of the contiguous input, perm[k] the input axis that becomes output axis k.
extern "C" int sb_canon_permute(const void* in, void* out, int rank, const long long* in_shape, const int* perm,
                                void* stream_) {
  if (rank < 1 || rank > 8 || !in || !out) return SB_ERR_ARG;
  long long in_stride[8], n = 1;
  unsigned seen = 0;
  for (int k = rank - 1; k >= 0; --k) {
    if (in_shape[k] <= 0) return SB_ERR_ARG;
    in_stride[k] = n;
    n *= in_shape[k];
  }
  PermuteArgs pa;
  pa.rank = rank;
  for (int k = 0; k < rank; ++k) {
    if (perm[k] < 0 || perm[k] >= rank || (seen & (1u << perm[k]))) return SB_ERR_ARG;
    seen |= 1u << perm[k];
    pa.out_shape[k] = in_shape[perm[k]];
    pa.in_stride[k] = in_stride[perm[k]];
  }
  canon_permute_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), n, pa);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
