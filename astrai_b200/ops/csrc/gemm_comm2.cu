// Tensor-parallel GEMMs fused with their collective, on the CTA-pair (tcgen05 cta_group::2) tile engine.
//
// Same two operations as gemm_comm.cu - all-gather -> GEMM and GEMM -> reduce-scatter over NVLink peer memory - built
// differently.  The tile engine is the 256x256 pair kernel of gemm_tcgen05_2cta.cu (each CTA loads its own 128 rows of
// A and half of B, 6-stage ring, accumulators double-buffered in TMEM), and the transfer does not take SMs away from
// it: every CTA has one extra warp whose elected lane moves 32 KB pieces with untiled bulk copies (peer memory ->
// shared memory -> local memory), one piece in flight per CTA, about 4.7 MB in flight per GPU - enough to keep
// NVLink busy while all 148 SMs multiply.
//
//   all-gather -> GEMM    Y[M, N] = concat_r(X_r)[M, K] * op(W).  Row block r of the local X_full is pulled from rank r
//       by the comm lanes (ring order, local block first needs no transfer); when the last CTA has stored its pieces of
//       a block it publishes chunk_flags[block]; the TMA producers walk the tiles block by block in the same order and
//       poll that flag (bounded) before the first load from a remote block.
//   GEMM -> reduce-scatter    Y_r[M/W, N] = sum_p (X_p * op(W_p))[row block r].  Every rank writes its whole partial
//       product into its own symmetric buffer with plain local stores (blocks in the order rank+1, rank+2, ..., own
//       block last) and tells the owner of a block when that block is complete; the comm lanes PULL the finished
//       blocks of the peers into a local staging buffer as they become available, overlapped with the remaining tiles;
//       at the end the epilogue warps sum the W partials in fp32 in a fixed order (deterministic).
// Bytes over NVLink are the same as for the push design of gemm_comm.cu, but they travel as 32 KB bulk copies instead
// of 64-byte stores, and the tensor pipe never waits for a remote store.
// No TMA multicast anywhere; TMA tensor loads only read this GPU's memory.  Every wait is bounded; expiry records a code
// in `status`, raises the CTA's abort flag and all roles leave through the common exit where TMEM is freed.
// The reference has no tensor parallelism (scripts/tools/train.py:513-519 parses --tp_size and drops it).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"
#include "flash_cp.cuh"
#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

using namespace tc;
using namespace tmah;
using namespace comm;
using cpx::bulk_commit;
using cpx::bulk_load;
using cpx::bulk_store;
using cpx::bulk_wait_all;
using cpx::bulk_wait_read;
using cpx::fence_async_global;
using cpx::flag_slot;
using cpx::ld_acquire_gpu;
using cpx::st_release_gpu;

constexpr int BM = 128, BN = 256, BNH = BN / 2, BK = 64, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KB
constexpr int PIECE = 32768;                                                                    // one bulk copy
constexpr int NUM_THREADS = 224;  // producer, MMA, 4 epilogue warps, comm warp
// Shared memory is split between the GEMM's operand ring (STAGES x 32 KB) and the comm lane's copy slots (SLOTS x 32 KB),
// seven 32 KB units in all: 6 + 1 (the default), 5 + 2 or 4 + 3.
constexpr int smem_bytes(int stages, int slots) { return (stages + slots) * STAGE_BYTES + 1024 + 256; }
enum : int { MODE_AG = 1, MODE_RS = 2 };
enum : int { ERR2_PRODUCER = 56, ERR2_MMA = 57, ERR2_EPILOGUE = 58, ERR2_COMM = 59, ERR2_REDUCE = 60 };
constexpr int KIND_AG = 2, KIND_RS = 3;  // flag planes (astrai_b200/parallel/symm.py)

__device__ __forceinline__ uint64_t make_desc2(uint32_t saddr, bool kmajor) {
  const uint64_t lbo = kmajor ? 1ull : (uint64_t)((BK * 128) >> 4);
  const uint64_t sbo = 1024 >> 4;
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

// Tile t -> (m0 of the pair tile, n0, row block).  Blocks are visited starting at `first_block`; inside a block groups
// of 8 pair-rows sweep all column tiles (the rasterisation of the plain pair kernel, applied per block).
struct Tile2 { int m0, n0, block; };
__device__ __forceinline__ Tile2 tile_of(int t, int tiles_m_blk, int tiles_n, int world, int first_block, int Ms) {
  const int per_block = tiles_m_blk * tiles_n;
  const int bi = t / per_block, r0 = t % per_block;
  const int block = (first_block + bi) % world;
  constexpr int G = 8;
  const int per_group = G * tiles_n;
  const int g = r0 / per_group, r = r0 % per_group;
  const int rows = min(G, tiles_m_blk - g * G);
  return {block * Ms + (g * G + r % rows) * (2 * BM), (r / rows) * BN, block};
}

// Move `bytes` (a multiple of 16) from `src` (possibly a peer's memory) to local `dst`: this CTA's share of the 32 KB
// pieces (piece index cta, cta + n_ctas, ...) through SLOTS shared-memory slots, so that up to SLOTS peer reads are in
// flight while an earlier piece is written out.  `phases` holds one parity bit per slot's mbarrier and lives across calls.
template <int SLOTS>
__device__ __forceinline__ bool copy_share(const uint8_t* src, uint8_t* dst, long long bytes, int cta, int n_ctas,
                                           uint32_t slot0, uint32_t bar0, uint32_t& phases, volatile int* abort_flag) {
  const long long n_pieces = (bytes + PIECE - 1) / PIECE;
  const long long mine = cta < n_pieces ? (n_pieces - cta + n_ctas - 1) / n_ctas : 0;
  auto off_of = [&](long long k) { return (cta + k * n_ctas) * (long long)PIECE; };
  auto len_of = [&](long long k) { return (uint32_t)min((long long)PIECE, bytes - off_of(k)); };
  auto issue = [&](long long k) {
    const int s = (int)(k % SLOTS);
    mbar_expect_tx(bar0 + 8u * s, len_of(k));
    bulk_load(slot0 + (uint32_t)s * PIECE, src + off_of(k), len_of(k), bar0 + 8u * s);
  };
  for (long long k = 0; k < mine && k < SLOTS; ++k) issue(k);
  for (long long k = 0; k < mine; ++k) {
    const int s = (int)(k % SLOTS);
    if (!mbar_wait(bar0 + 8u * s, (phases >> s) & 1u, abort_flag)) return false;
    phases ^= 1u << s;
    bulk_store(dst + off_of(k), slot0 + (uint32_t)s * PIECE, len_of(k));
    bulk_commit();
    if (k + SLOTS < mine) {
      bulk_wait_read();  // the store has read the slot: the next peer read may land in it
      issue(k + SLOTS);
    }
  }
  bulk_wait_all();  // every store of this share has landed
  return true;
}

// out[v] = sum over the W sources of their vector v (fp32 accumulation, bf16 in and out); source `rank` is `own`, source
// s != rank is slot s of `gath`.  VPT adjacent vectors of every source per thread and trip; W <= WMAX.
template <int VPT, int WMAX>
__device__ __forceinline__ void reduce_slots(const __nv_bfloat16* own, const __nv_bfloat16* gath, void* out, int W, int rank,
                                             long long slot_elems, long long n_vec, long long tid, long long nthr) {
  for (long long v = VPT * tid; v < n_vec; v += VPT * nthr) {
    uint4 raw[WMAX][VPT];
#pragma unroll
    for (int s = 0; s < WMAX; ++s) {
      if (s < W) {
        const __nv_bfloat16* src = (s == rank) ? own : gath + (long long)s * slot_elems;
#pragma unroll
        for (int u = 0; u < VPT; ++u) raw[s][u] = __ldcg(reinterpret_cast<const uint4*>(src) + v + u);
      }
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < WMAX; ++s) {
        if (s < W) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[s][u]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(h[q]);
            acc[2 * q] += f.x, acc[2 * q + 1] += f.y;
          }
        }
      }
      uint4 pk;
      uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
        pw[q] = *reinterpret_cast<const uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(out)[v + u] = pk;
    }
  }
}

template <int MODE, bool B_K, int STAGES, int SLOTS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_comm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  __nv_bfloat16* __restrict__ D, int M, int N, int K, long long ldd, const TpGemmParams p,
                  int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t slot = base + STAGES * STAGE_BYTES;  // the comm lane's 32 KB pieces
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (STAGES + SLOTS) * STAGE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  const uint32_t copy_bar = bar0 + 8u * (2 * STAGES + 4);  // SLOTS barriers, one per copy slot
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();  // 0 = leader of the pair
  const bool leader = crank == 0;
  const int W = p.world, Ms = M / W;
  const int tiles_m_blk = Ms / (2 * BM), tiles_n = (N + BN - 1) / BN, per_block = tiles_m_blk * tiles_n;
  const int num_tiles = per_block * W, num_kb = (K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int cta = blockIdx.x, n_ctas = gridDim.x;
  const int first_block = (MODE == MODE_RS) ? (p.rank + 1) % W : p.rank;
  const bool do_gemm = !(MODE == MODE_RS && p.fuse_reduce == 2);   // 2: pull + reduce only (single-GPU emulation)
  const bool do_pull = !(MODE == MODE_RS && p.fuse_reduce == 0);   // 0: product + announcements only

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);  // 4 epilogue warps x 2 CTAs arrive on the leader's copy
    }
    for (int c = 0; c < SLOTS; ++c) mbar_init(copy_bar + 8u * c, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0 && do_gemm) {
      int stage = 0, ready_block = -1;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const Tile2 tl = tile_of(t, tiles_m_blk, tiles_n, W, first_block, Ms);
        if (MODE == MODE_AG && tl.block != p.rank && tl.block != ready_block) {
          const unsigned long long t0 = now_ns();
          while (ld_acquire_gpu(&p.chunk_flags[tl.block]) < p.epoch) {
            if (*abort_flag || now_ns() - t0 > p.timeout_ns) {
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_async_global();  // the rows were written by bulk stores and are read by TMA
          ready_block = tl.block;
        }
        const int m0 = tl.m0 + (int)crank * BM, n0 = tl.n0 + (int)crank * BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint32_t fb = mapa(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_2d_cg2(sa, &map_a, fb, k0, m0);
          if (B_K) {
            tma_load_2d_cg2(sb, &map_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_cg2(sb + j * (BK * 128), &map_b, fb, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR2_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0 && do_gemm) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((B_K ? 0u : 1u) << 16) |
                                 ((uint32_t)((2 * BM) >> 4) << 24) | ((uint32_t)(BN >> 3) << 17);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t da = make_desc2(sa, true), db = make_desc2(sb, B_K);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ka = (uint64_t)((k * UMMA_K * 2) >> 4);
            const uint64_t kbo = (uint64_t)((B_K ? k * UMMA_K * 2 : k * UMMA_K * 128) >> 4);
            tc_mma_cg2(d_tmem, da + ka, db + kbo, idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit_cg2(empty_bar(stage), 3);
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) tc_commit_cg2(tfull_bar(buf), 3);
      }
      if (!ok) {
        atomicMax(status, ERR2_MMA);
        *abort_flag = 1;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (both CTAs), then the reduce phase
    const int quarter = warp & 3;
    const uint32_t tempty_leader0 = mapa(tempty_bar(0), 0), tempty_leader1 = mapa(tempty_bar(1), 0);
    int it = 0;
    bool ok = true;
    for (int t = pair; do_gemm && t < num_tiles && ok; t += num_pairs, ++it) {
      const int buf = it & 1;
      const Tile2 tl = tile_of(t, tiles_m_blk, tiles_n, W, first_block, Ms);
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tl.m0 + (int)crank * BM + quarter * 32 + lane;
      __nv_bfloat16* drow = D + (long long)row * ldd;  // AG: the output; RS: this rank's partial product [M, N]
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld32(taddr0 + c * 32, r);
        tc_wait_ld();
        const int col = tl.n0 + c * 32;
        if (row < M && col + 32 <= N) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 pk;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * q]), __uint_as_float(r[8 * j + 2 * q + 1]));
              pw[q] = *reinterpret_cast<const uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(drow + col)[j] = pk;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? tempty_leader1 : tempty_leader0);  // the accumulator is free at once
      if (MODE == MODE_RS) {
        // count warp arrivals per row block; the last one tells the block's owner that this rank's partial is complete.
        // Every warp orders its stores before its arrival at GPU scope; the last arriver's system-scope fence then
        // carries all of them to the peer together with the flag (fences are cumulative).
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          const int done = atomicAdd(&p.tile_counter[tl.block], 1);
          if (done == 8 * per_block - 1) {
            __threadfence_system();
            st_release_sys(flag_slot(p.flags[tl.block], KIND_RS, p.rank, p.unit, p.max_units), p.epoch);
          }
        }
      }
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR2_EPILOGUE);
      *abort_flag = 1;
    }
    if (MODE == MODE_RS && ok && do_pull) {
      // ---- reduce phase: every CTA's comm lane has pulled its share of the peers' blocks, and the own block is complete
      bool got = true;
      if (lane == 0) {
        const unsigned long long t0 = now_ns();
        while (ld_acquire_gpu(p.pull_counter) < n_ctas) {
          if (*abort_flag || now_ns() - t0 > p.timeout_ns) {
            got = false;
            break;
          }
          __nanosleep(200);
        }
        if (got) got = wait_flag(flag_slot(p.flags[p.rank], KIND_RS, p.rank, p.unit, p.max_units), p.epoch, p.timeout_ns);
      }
      got = __all_sync(0xffffffffu, got);
      if (!got) {
        if (lane == 0) atomicMax(status, ERR2_REDUCE);
      } else {
        const long long slot_elems = (long long)Ms * N, n_vec = slot_elems / 8;
        const __nv_bfloat16* own = reinterpret_cast<const __nv_bfloat16*>(p.stage[p.rank]) + (long long)p.rank * slot_elems;
        const __nv_bfloat16* gath = reinterpret_cast<const __nv_bfloat16*>(p.gathered);
        const long long tid = (long long)cta * 128 + (warp - 2) * 32 + lane, nthr = (long long)n_ctas * 128;
        // About 16 independent 16-byte loads per thread and trip, all issued before the first add, whatever the number
        // of ranks: with few sources a thread takes more vectors of each (the sum then runs at memory speed instead of
        // at one load latency per trip).  N is a multiple of 32 and Ms of 256, so the vector count divides by 8.
        if (W <= 2) reduce_slots<8, 2>(own, gath, p.rs_out, W, p.rank, slot_elems, n_vec, tid, nthr);
        else if (W <= 4) reduce_slots<4, 4>(own, gath, p.rs_out, W, p.rank, slot_elems, n_vec, tid, nthr);
        else reduce_slots<2, MAX_RANKS>(own, gath, p.rs_out, W, p.rank, slot_elems, n_vec, tid, nthr);
      }
    }
  } else {
    // ------------------------------------------------------------ comm warp: bulk copies peer -> shared -> local
    if (lane == 0) {
      bool ok = true;
      uint32_t cphase = 0;
      if (MODE == MODE_AG) {
        if (cta == 0) {  // this rank's own block was placed in X_full before the launch: announce it to everybody
          __threadfence_system();
          for (int q = 0; q < W; ++q) st_release_sys(flag_slot(p.flags[q], KIND_AG, p.rank, p.unit, p.max_units), p.epoch);
        }
        const long long blk_bytes = (long long)Ms * K * 2;
        for (int i = 1; i < W && ok; ++i) {
          const int src = (p.rank + i) % W;
          if (!wait_flag(flag_slot(p.flags[p.rank], KIND_AG, src, p.unit, p.max_units), p.epoch, p.timeout_ns)) {
            ok = false;
            break;
          }
          const uint8_t* from = reinterpret_cast<const uint8_t*>(p.x_full[src]) + (long long)src * blk_bytes;
          uint8_t* to = reinterpret_cast<uint8_t*>(p.x_full[p.rank]) + (long long)src * blk_bytes;
          ok = copy_share<SLOTS>(from, to, blk_bytes, cta, n_ctas, slot, copy_bar, cphase, abort_flag);
          if (!ok) break;
          fence_async_global();
          __threadfence();
          const int done = atomicAdd(&p.chunk_counter[src], 1);
          if (done == n_ctas - 1) {
            p.chunk_counter[src] = 0;
            st_release_gpu(&p.chunk_flags[src], p.epoch);
          }
        }
      } else if (do_pull) {
        const long long blk_bytes = (long long)Ms * N * 2;
        for (int i = 0; i < W - 1 && ok; ++i) {
          const int src = (p.rank - 1 - i + 2 * W) % W;  // the peer that finishes this rank's block earliest comes first
          if (!wait_flag(flag_slot(p.flags[p.rank], KIND_RS, src, p.unit, p.max_units), p.epoch, p.timeout_ns)) {
            ok = false;
            break;
          }
          const uint8_t* from = reinterpret_cast<const uint8_t*>(p.stage[src]) + (long long)p.rank * blk_bytes;
          uint8_t* to = reinterpret_cast<uint8_t*>(p.gathered) + (long long)src * blk_bytes;
          ok = copy_share<SLOTS>(from, to, blk_bytes, cta, n_ctas, slot, copy_bar, cphase, abort_flag);
        }
        if (ok) {
          fence_async_global();
          __threadfence();
          atomicAdd(p.pull_counter, 1);
        }
      }
      if (!ok) {
        atomicMax(status, ERR2_COMM);
        *abort_flag = 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

template <int MODE, bool B_K, int STAGES, int SLOTS>
int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd, const TpGemmParams& p,
               int* status, cudaStream_t st) {
  auto kern = gemm2_comm_kernel<MODE, B_K, STAGES, SLOTS>;
  constexpr int SMEM = smem_bytes(STAGES, SLOTS);
  static bool configured = false;
  static int max_pairs = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -4;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sms / 2;
    }
    max_pairs = clusters < sms / 2 ? clusters : sms / 2;
    configured = true;
  }
  // every CTA must be resident at once (the roles wait on one another's flags and every CTA carries a share of the
  // transfer): never more pairs than fit, and all of them even when there are fewer tiles
  const int tiles = (M / (2 * BM)) * ((N + BN - 1) / BN);
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, NUM_THREADS, SMEM, st>>>(ma, mb, (__nv_bfloat16*)D, M, N, K, ldd, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Copy slots when the caller does not name a number.  Measured on 8 B200s (65 536 tokens, the 8B model's four projection
// shapes, 1 / 3 slots): 1.69 / 2.11 ms, 0.93 / 1.77 ms, 1.04 / 1.51 ms, 1.03 / 1.86 ms - the operand stages given up cost
// the GEMM more than the extra bytes in flight give the transfer, for compute-bound and link-bound shapes alike.  So the
// default is one slot and six stages; 2 and 3 remain selectable per call.
int copy_slots(int /*M*/, int /*N*/, int /*K*/, int /*world*/, bool /*rs*/) { return 1; }

template <int MODE, bool B_K>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd, const TpGemmParams& p,
           int* status, cudaStream_t st) {
  int slots = p.copy_slots > 0 ? p.copy_slots : copy_slots(M, N, K, p.world, MODE == MODE_RS);
  if (slots >= 3) return launch_cfg<MODE, B_K, 4, 3>(ma, mb, D, M, N, K, ldd, p, status, st);
  if (slots == 2) return launch_cfg<MODE, B_K, 5, 2>(ma, mb, D, M, N, K, ldd, p, status, st);
  return launch_cfg<MODE, B_K, 6, 1>(ma, mb, D, M, N, K, ldd, p, status, st);
}

int check(const TpGemmParams& p, int M, int N, int K) {
  if (p.world < 1 || p.world > MAX_RANKS || p.rank < 0 || p.rank >= p.world) return -1;
  if (M % (p.world * 2 * BM) || N % 32 || K % 8) return -2;  // row blocks are whole pair tiles; 32-column epilogue chunks
  if (p.unit < 0 || p.unit >= p.max_units) return -3;
  return 0;
}

}  // namespace

bool tp2_shape_ok(int M, int N, int K, int world) { return world >= 1 && M % (world * 2 * BM) == 0 && N % 32 == 0 && K % 8 == 0; }

int gemm_allgather2(const void* W, bool w_kmajor, void* Y, int M, int N, int K, long long ldy, const TpGemmParams& p,
                    int* status, cudaStream_t st) {
  if (int rc = check(p, M, N, K)) return rc;
  if (!p.chunk_flags || !p.chunk_counter) return -6;
  CUtensorMap ma, mb;
  if (!cache().get(&ma, p.x_full[p.rank], K, M, K, BK, BM)) return -1000 - g_last_map_error;
  const bool okb = w_kmajor ? cache().get(&mb, W, K, N, K, BK, BNH) : cache().get(&mb, W, N, K, N, 64, BK);
  if (!okb) return -2000 - g_last_map_error;
  return w_kmajor ? launch<MODE_AG, true>(ma, mb, Y, M, N, K, ldy, p, status, st)
                  : launch<MODE_AG, false>(ma, mb, Y, M, N, K, ldy, p, status, st);
}

int gemm_reducescatter2(const void* X, const void* W, bool w_kmajor, int M, int N, int K, const TpGemmParams& p,
                        int* status, cudaStream_t st) {
  if (int rc = check(p, M, N, K)) return rc;
  if (!p.tile_counter || !p.pull_counter || !p.gathered || !p.rs_out) return -6;
  CUtensorMap ma, mb;
  if (!cache().get(&ma, X, K, M, K, BK, BM)) return -1000 - g_last_map_error;
  const bool okb = w_kmajor ? cache().get(&mb, W, K, N, K, BK, BNH) : cache().get(&mb, W, N, K, N, 64, BK);
  if (!okb) return -2000 - g_last_map_error;
  if (p.fuse_reduce != 2 && cudaMemsetAsync(p.tile_counter, 0, sizeof(int) * MAX_RANKS, st) != cudaSuccess) return -7;
  if (cudaMemsetAsync(p.pull_counter, 0, sizeof(int), st) != cudaSuccess) return -7;
  void* part = p.stage[p.rank];  // this rank's partial product [M, N]
  return w_kmajor ? launch<MODE_RS, true>(ma, mb, part, M, N, K, N, p, status, st)
                  : launch<MODE_RS, false>(ma, mb, part, M, N, K, N, p, status, st);
}

}  // namespace ab
