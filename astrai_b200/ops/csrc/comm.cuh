// Device-side communication primitives over NVLink peer memory and NVSwitch multicast (NVLS) addresses.
//
// Peer pointers come from one symmetric allocation per rank that is mapped into every rank of the node
// (astrai_b200/parallel/symm.py).  Signalling is flag based: the writer stores a monotonically increasing epoch
// with release semantics at system scope, the reader polls with acquire loads.  EVERY wait is bounded by a
// globaltimer budget; a wait that runs out records an error code in the status word and the kernel returns
// without touching the data, so the context stays usable and the host can raise.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ab {
namespace comm {

constexpr int MAX_RANKS = 8;

enum : int { ERR_WAIT_PEER_READY = 21, ERR_WAIT_PEER_DONE = 22, ERR_WAIT_FLAG = 23 };

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Coherent 16-byte load of (possibly remote) memory: never served from a stale L1 line.
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// In-switch reduction: one load returns the sum of the addressed 16 bytes over every rank bound to the multicast object.
__device__ __forceinline__ float4 mc_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// In-switch broadcast: one store lands in every rank's copy.
__device__ __forceinline__ void mc_st_u4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Poll until *flag >= epoch.  False when the budget ran out.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, unsigned long long timeout_ns) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const unsigned long long t0 = now_ns();
  for (unsigned spin = 1;; ++spin) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if ((spin & 15u) == 0) {
      if (now_ns() - t0 > timeout_ns) return false;
      __nanosleep(200);
    }
  }
}

}  // namespace comm
}  // namespace ab
