// Flag protocol helpers shared by the kernels that talk to other GPUs through peer-mapped memory
// (comm.cu, decode.cu): system-scope release stores and acquire loads on epoch words, bounded waits that
// record ST_TIMEOUT_PEER in the status word instead of spinning for ever, and the 16-byte volatile peer load.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "sm100_ptx.cuh"

namespace sb {

constexpr int MAX_WORLD = 16;
constexpr int SLOT_WORDS = 4 * MAX_WORLD;  // flag words per slot (phases 0..3 x MAX_WORLD ranks)
constexpr uint64_t kPeerWaitNsDefault = 10000000000ull;  // 10 s: a peer may start its kernel late

struct PeerTable {
  void* in[MAX_WORLD];        // peers' input buffers (bucket base)
  void* out[MAX_WORLD];       // peers' output buffers
  uint32_t* flags[MAX_WORLD]; // peers' flag arrays
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Wait until flags[0..W-1] >= epoch (epochs only grow). One thread calls this.
__device__ inline bool wait_flags(const uint32_t* flags, int W, uint32_t epoch, uint64_t limit_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  for (int r = 0; r < W; ++r) {
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flags + r) - epoch) < 0) {
      if ((++spins & 0xff) == 0) {
        if (globaltimer_ns() - t0 > limit_ns) {
          atomicCAS(status, 0, ST_TIMEOUT_PEER);
          return false;
        }
        if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      }
    }
  }
  return true;
}

// Wait until flags[0..W-1] >= epoch with lanes 0..W-1 of the calling warp polling one flag each (W <= 16).
// Every lane of the warp must call it; returns the same verdict on all lanes.
__device__ inline bool wait_flags_warp(const uint32_t* flags, int W, uint32_t epoch, uint64_t limit_ns, int* status) {
  const int lane = threadIdx.x & 31;
  const uint64_t t0 = globaltimer_ns();
  bool ok = true;
  if (lane < W) {
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flags + lane) - epoch) < 0) {
      if ((++spins & 0xff) == 0) {
        if (globaltimer_ns() - t0 > limit_ns) {
          atomicCAS(status, 0, ST_TIMEOUT_PEER);
          ok = false;
          break;
        }
        if (*reinterpret_cast<volatile int*>(status) != 0) { ok = false; break; }
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}

}  // namespace sb
