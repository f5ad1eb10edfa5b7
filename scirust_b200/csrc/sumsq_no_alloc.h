// Sum of squares without any allocation.
//
// This entry point has no counterpart in the reference; it exists for hosts that cannot
// allocate device memory at the moment they need a gradient norm. Two kinds of caller are in
// that position: a program that has already handed all free device memory to its own pool, so
// a cudaMalloc for a few kilobytes of scratch would simply fail; and a latency-sensitive loop
// that must not pay for cudaMalloc/cudaFree, which take a driver lock and can synchronise the
// whole device. `sb_sumsq` asks such callers for a scratch buffer they may not have;
// `sb_sumsq_no_alloc` brings its own.
//
// The scratch is one array that lives inside the library image
// (SB_SUMSQ_NO_ALLOC_MAX_PARTIALS floats = 256 KiB, held on every GPU that loads the library
// until the process exits). That bounds the input: at most SB_SUMSQ_NO_ALLOC_MAX_ELEMS
// elements per call; a longer input is refused with SB_ERR_TOO_LARGE and nothing is launched.
//
// Rules of use:
//  * The first call on each device looks up the device address of the array (no allocation,
//    but a runtime query). Make that first call before any stream capture begins.
//  * All calls on a device share the one array. A call overwrites exactly the partials it later
//    reads, so nothing has to be cleared beforehand and stale contents are harmless; but two
//    calls whose kernels overlap on the GPU (different streams, no ordering between them) race
//    on the array and both results are then undefined. Keep calls on one stream or order them.
//  * The result is bit-identical to `sb_sumsq` on the same input: the same two kernels run with
//    the same launch shape, only the scratch comes from a different place.
#pragma once
#include <stddef.h>

#define SB_SUMSQ_NO_ALLOC_MAX_PARTIALS 65536
#define SB_SUMSQ_NO_ALLOC_ELEMS_PER_PARTIAL 4096
#define SB_SUMSQ_NO_ALLOC_MAX_ELEMS \
  ((size_t)SB_SUMSQ_NO_ALLOC_MAX_PARTIALS * (size_t)SB_SUMSQ_NO_ALLOC_ELEMS_PER_PARTIAL)

#ifdef __cplusplus
extern "C" {
#endif

// g: n elements, bf16 (is_bf16 != 0) or fp32, on the current device. out: one fp32 on the same
// device; receives the sum of squares, or has it added when accumulate != 0. Returns 0, or
// SB_ERR_ARG (n == 0, null pointer), SB_ERR_TOO_LARGE (n > SB_SUMSQ_NO_ALLOC_MAX_ELEMS),
// SB_ERR_RUNTIME (the scratch address could not be resolved), SB_ERR_LAUNCH.
int sb_sumsq_no_alloc(const void* g, size_t n, int is_bf16, float* out, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
