// Expert-parallel routing exchange: who sends how many rows to which expert, and where each row lands.
//
// E experts are split evenly over the ranks (rank d owns experts [d * El, (d + 1) * El)).  After the local router every
// rank knows, per expert, how many of ITS (token, choice) pairs go there.  Two small single-CTA kernels turn that into
// a plan every rank agrees on without a host round trip or a collective call:
//   ep_push_counts : the local counts row is stored into every peer's counts table over NVLink, the local row table is
//                    blanked, and a flag is published.
//   ep_plan        : waits (bounded) for every rank's counts; lays out, for EVERY rank d, the segments of its experts
//                    (rows of source rank 0 first, then rank 1, ...; each segment padded to 128 rows) - the same
//                    arithmetic on every rank, so no offsets need to travel; writes the local segment offsets and tile
//                    map for the grouped GEMM; then claims a slot for each local (token, choice) pair and stores
//                    `rank << 24 | pair` into the owner's row table.  The rows themselves never move here: the
//                    grouped GEMM pulls them (gemm_grouped.cu, EpRows).
// The reference has no expert parallelism (its MoE loops over experts on one device,
// astrai/model/components/mlp.py:143-166).
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"
#include "launchers.h"

namespace ab {
namespace {

using namespace comm;

constexpr int KIND_EP = 5;  // flag plane (astrai_b200/parallel/symm.py)
constexpr int MAX_E = 256;
enum : int { ERR_EP_PLAN_WAIT = 71, ERR_EP_OVERFLOW = 72 };

struct Ptrs8 { void* p[8]; };

__device__ __forceinline__ int* flag_slot(void* base, int kind, int src, int unit, int max_units) {
  return reinterpret_cast<int*>(base) + ((long long)kind * MAX_RANKS + src) * max_units + unit;
}

__global__ void ep_push_counts_kernel(const int* __restrict__ counts_local, int E, Ptrs8 counts_all, int* __restrict__ row_peer_local,
                                      int r_cap, Ptrs8 flags, int world, int rank, int unit, int max_units, int epoch) {
  for (int i = threadIdx.x; i < r_cap; i += blockDim.x) row_peer_local[i] = -1;
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int p = i / E, e = i % E;
    reinterpret_cast<int*>(counts_all.p[p])[rank * E + e] = counts_local[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(flag_slot(flags.p[threadIdx.x], KIND_EP, rank, unit, max_units), epoch);
}

__global__ void ep_plan_kernel(const long long* __restrict__ idx, long long pairs, const int* __restrict__ counts_all, Ptrs8 row_peer,
                               int* __restrict__ offsets, int* __restrict__ tile_expert, int* __restrict__ total, int E, int r_cap,
                               Ptrs8 flags, int world, int rank, int wait_unit, int signal_unit, int max_units, int epoch,
                               unsigned long long timeout_ns, int* __restrict__ status) {
  __shared__ int s_cnt[MAX_RANKS * MAX_E];  // counts[src][e]
  __shared__ int s_base[MAX_E];             // first row of THIS rank's pairs inside expert e's segment on its owner
  __shared__ int s_cursor[MAX_E];
  __shared__ int s_off[MAX_E + 1];          // local padded segment offsets
  __shared__ int s_ok;
  const int El = E / world;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int src = 0; src < world && ok; ++src)
      ok = wait_flag(flag_slot(flags.p[rank], KIND_EP, src, wait_unit, max_units), epoch, timeout_ns) ? 1 : 0;
    if (!ok) atomicMax(status, ERR_EP_PLAN_WAIT);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  for (int i = threadIdx.x; i < world * E; i += blockDim.x)
    s_cnt[i] = ld_acquire_sys(counts_all + i);  // written by the peers over NVLink: never from a stale line
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_cursor[e] = 0;
  __syncthreads();
  // one thread per owner rank d: walk its experts, padded segment by padded segment
  if (threadIdx.x < world) {
    const int d = threadIdx.x;
    int off = 0;
    for (int le = 0; le < El; ++le) {
      const int e = d * El + le;
      int n = 0, before_me = 0;
      for (int src = 0; src < world; ++src) {
        if (src == rank) before_me = n;
        n += s_cnt[src * E + e];
      }
      s_base[e] = off + before_me;
      if (d == rank) s_off[le] = off;
      off += (n + 127) / 128 * 128;
    }
    if (d == rank) s_off[El] = off;
    if (off > r_cap) atomicMax(status, ERR_EP_OVERFLOW), s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;  // a row table would overflow: nothing is entered, the flag is not published, the peers time out
  for (int le = threadIdx.x; le <= El; le += blockDim.x) offsets[le] = s_off[le];
  if (threadIdx.x == 0) *total = s_off[El];
  for (int t = threadIdx.x; t < r_cap / 128; t += blockDim.x) {
    const int row = t * 128;
    int lo = 0, hi = El;  // last le with s_off[le] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_off[mid] <= row) lo = mid; else hi = mid;
    }
    tile_expert[t] = (row < s_off[El] && row < s_off[lo + 1]) ? lo : -1;
  }
  for (long long w = threadIdx.x; w < pairs; w += blockDim.x) {
    const int e = (int)idx[w];
    const int slot = s_base[e] + atomicAdd(&s_cursor[e], 1);
    reinterpret_cast<int*>(row_peer.p[e / El])[slot] = (rank << 24) | (int)w;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(flag_slot(flags.p[threadIdx.x], KIND_EP, rank, signal_unit, max_units), epoch);
}

Ptrs8 pack(void* const* p, int n) {
  Ptrs8 r{};
  for (int i = 0; i < n && i < 8; ++i) r.p[i] = p[i];
  return r;
}

}  // namespace

int ep_push_counts(const int* counts_local, int E, void* const* counts_all, int* row_peer_local, int r_cap, void* const* flags,
                   int world, int rank, int unit, int max_units, int epoch, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || E < world || E > MAX_E || E % world || r_cap % 128) return -1;
  ep_push_counts_kernel<<<1, 1024, 0, st>>>(counts_local, E, pack(counts_all, world), row_peer_local, r_cap, pack(flags, world), world,
                                            rank, unit, max_units, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ep_plan(const long long* idx, long long pairs, const int* counts_all_local, void* const* row_peer, int* offsets,
            int* tile_expert, int* total, int E, int r_cap, void* const* flags, int world, int rank, int wait_unit,
            int signal_unit, int max_units, int epoch, unsigned long long timeout_ns, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || E < world || E > MAX_E || E % world || r_cap % 128) return -1;
  if (pairs >= (1 << 24)) return -2;  // a pair index must fit beside the rank in one int
  ep_plan_kernel<<<1, 1024, 0, st>>>(idx, pairs, counts_all_local, pack(row_peer, world), offsets, tile_expert, total, E, r_cap,
                                     pack(flags, world), world, rank, wait_unit, signal_unit, max_units, epoch, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
