// Device-side pieces of context-parallel (sequence-sharded) flash attention that the forward and backward kernels
// share: the zig-zag chunk geometry, the order in which one CTA visits its key tiles, flag helpers and the bulk-copy
// instructions of the gather CTAs.
//
// Geometry (see CpAttn in launchers.h): S = 2 * W * c tokens in 2W chunks; rank r owns chunks r and 2W - 1 - r, stored
// locally as rows [0, c) and [c, 2c).  Chunk ch is owned by rank ch (ch < W) or 2W - 1 - ch.
// The reference has no sequence-parallel attention; its parallel package stops at data parallelism
// (astrai/parallel/setup.py:44-90).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"
#include "launchers.h"

namespace ab {
namespace cpx {

constexpr int KIND_CP_KV = 4, KIND_CP_DKV = 6;  // flag planes (astrai_b200/parallel/symm.py)
enum : int { ERR_CP_COPY = 61, ERR_CP_CHUNK_WAIT = 62, ERR_CP_REDUCE = 63 };

__device__ __forceinline__ int chunk_owner(int ch, int W) { return ch < W ? ch : 2 * W - 1 - ch; }
// Global chunk index of local half `half` (0: rows [0, c), 1: rows [c, 2c)) of rank p.
__device__ __forceinline__ int chunk_of(int p, int half, int W) { return half ? 2 * W - 1 - p : p; }

__device__ __forceinline__ int* flag_slot(void* base, int kind, int src, int unit, int max_units) {
  return reinterpret_cast<int*>(base) + ((long long)kind * comm::MAX_RANKS + src) * max_units + unit;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Untiled bulk copies (TMA without a tensor map): global -> shared with mbarrier completion, shared -> global in a
// bulk group.  Both addresses 16-byte aligned, size a multiple of 16.  The source may be a peer's memory; no multicast.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// The order in which a CTA visits its n_kv key tiles of `tile` keys each.  Plain attention: 0, 1, 2, ...  Context
// parallel: by owner in ring order starting with this rank (its own chunks need no transfer, then the chunks arrive in
// the order the gather CTAs pull them), both chunks of an owner, tiles of a chunk in ascending order.  Every tile
// below n_kv is visited exactly once; the softmax is order independent.
struct KvOrder {
  int n_kv, tpc, W, r, i, half, t, lin;
  __device__ KvOrder(int n_kv_, const CpAttn& cp, int tile) : n_kv(n_kv_), W(cp.world), r(cp.rank), i(0), half(0), t(0), lin(0) {
    tpc = cp.world > 1 ? cp.chunk / tile : 0;
  }
  __device__ int next() {
    if (W <= 1) return lin < n_kv ? lin++ : -1;
    while (i < W) {
      const int o = (r + i) % W;
      const int j = chunk_of(o, half, W) * tpc + t;
      if (t < tpc && j < n_kv) {
        ++t;
        return j;
      }
      t = 0;
      if (++half == 2) half = 0, ++i;
    }
    return -1;
  }
};

}  // namespace cpx
}  // namespace ab
