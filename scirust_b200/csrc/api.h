// Public C ABI of libscirust_b200_cuda.so. Python reaches these through ctypes
// (scirust_b200/ops/_lib.py); every entry point takes raw device pointers plus the
// CUDA stream to launch on, allocates nothing unless stated, and returns 0 or an
// SB_ERR_* code. Kernels that can wait (mbarrier / peer flags) also take a device
// `status` word: they store an sb::ST_* code there when a bounded wait runs out.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define SB_ERR_ARG 1
#define SB_ERR_ALIGN 2
#define SB_ERR_DRIVER 3
#define SB_ERR_LAUNCH 4
#define SB_ERR_TOO_LARGE 5
#define SB_ERR_RUNTIME 6

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM (gemm_tcgen05.cu) ---------------------------------------------------
int sb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                 int ldc, int ldr, int a_mn, int b_mn, int splits, void* workspace, int bn, int* status,
                 void* stream);

#ifdef __cplusplus
}
#endif
