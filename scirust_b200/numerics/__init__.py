"""Determinism toolkit: correctly rounded order-independent sums and dot products, a long
accumulator, libm-free bit-portable exp/ln/tanh/softmax/GEMM, bf16/f16/fp8 codecs."""
