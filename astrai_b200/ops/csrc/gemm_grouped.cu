// Grouped (per-expert) bf16 GEMMs for mixture-of-experts layers on tcgen05, driven by device-side segment tables.
//
// Tokens arrive expert-sorted in segments padded to 128 rows (moe.cu::moe_plan), so a 128-row tile belongs to exactly
// one expert and the row count per expert never has to reach the host.
//   rows mode  : Y[r, :] = X[r, :] . op(W_e) for every row r of expert e's segment.  The tile -> expert map selects the
//                row block of the stacked weight (K-major [N, K] per expert for the forward projection, MN-major
//                [Kc, N] per expert for the input gradient).  Tiles past the last segment are skipped by all roles.
//   wgrad mode : dW_e[N, K] (+)= dY_e^T . X_e, the contraction running over the rows of expert e's segment only
//                (ragged K read from the offsets table); both operands are MN-major views of the sorted buffers.
// Expert weights may live in one flat buffer with a fixed row stride per expert (gate|up|down interleaved), so no
// stacking copy is needed.  Structure and barriers follow gemm_tcgen05.cu (persistent, TMA ring, one MMA lane,
// double-buffered TMEM accumulator, four epilogue warps); all waits are bounded.
// Expert parallel (EpRows, rows mode): the sorted rows belong to tokens of other ranks.  Gather: copy CTAs at the front
// of the grid pull each 128-row tile's rows from the peers' memory (one bulk copy per row through shared memory, two
// batches in flight), zero the padding and publish a per-tile flag that the TMA producer of the GEMM CTAs polls - the
// all-to-all dispatch overlaps the expert GEMM tile by tile.  Scatter: the epilogue stores every output row straight
// into the memory of the rank that owns the token (the combine all-to-all), the last CTA publishes a flag.
// Replaces the reference's Python loop over experts (astrai/model/components/mlp.py:143-166).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flash_cp.cuh"
#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

using namespace tc;
using namespace tmah;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
enum : int { MODE_ROWS = 0, MODE_WGRAD = 1 };
enum : int { ERR_GG_PRODUCER = 81, ERR_GG_MMA = 82, ERR_GG_EPILOGUE = 83, ERR_GG_GATHER = 84, ERR_GG_TILE_WAIT = 85 };
constexpr int KIND_EP = 5;  // flag plane (astrai_b200/parallel/symm.py)

// Copy CTA of the expert-parallel gather (all threads take part).  Tiles are dealt round-robin to the copy CTAs.
__device__ void ep_gather(const EpRows& ep, int cta, int n_copy, int R, int K, uint8_t* a_local, const int* tile_expert,
                          int* status) {
  using namespace cpx;
  constexpr int HALF = STAGES * STAGE_BYTES / 2;  // two slots
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + 2 * HALF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2);
  __shared__ int s_ok;
  const uint32_t bar0 = smem_u32(bars);
  if (threadIdx.x == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
    if (cta == 0 && ep.announce_unit >= 0) {
      __threadfence_system();
      for (int p = 0; p < ep.world; ++p) comm::st_release_sys(flag_slot(ep.flags[p], KIND_EP, ep.rank, ep.announce_unit, ep.max_units), ep.epoch);
    }
    int ok = 1;
    for (int src = 0; src < ep.world && ok; ++src)
      ok = comm::wait_flag(flag_slot(ep.flags[ep.rank], KIND_EP, src, ep.wait_unit, ep.max_units), ep.epoch, ep.timeout_ns) ? 1 : 0;
    if (!ok) atomicMax(status, ERR_GG_GATHER);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;  // the GEMM CTAs run out of time on the tile flag and report as well
  const uint32_t row_bytes = (uint32_t)K * 2u;
  const int rps = min(128, (int)(HALF / row_bytes));  // rows per slot
  uint32_t uses[2] = {0, 0};
  for (int mt = cta; mt < R / 128; mt += n_copy) {
    if (tile_expert[mt] < 0) continue;
    const int* rp = ep.row_peer + mt * 128;
    const int nv = __syncthreads_count(threadIdx.x < 128 && comm::ld_acquire_sys(rp + min((int)threadIdx.x, 127)) >= 0);
    // padding rows (always the tail of a tile): zeros, so they add nothing to a weight gradient
    uint4* pad = reinterpret_cast<uint4*>(a_local + ((long long)mt * 128 + nv) * row_bytes);
    const long long n16 = (long long)(128 - nv) * (row_bytes / 16);
    for (long long i = threadIdx.x; i < n16; i += blockDim.x) pad[i] = make_uint4(0, 0, 0, 0);
    fence_async_global();
    __threadfence();
    if (threadIdx.x == 0) {
      const int nb = (nv + rps - 1) / rps;
      auto issue = [&](int b) {
        const int slot = b & 1, r0 = b * rps, n = min(rps, nv - r0);
        mbar_expect_tx(bar0 + 8u * slot, (uint32_t)n * row_bytes);
        for (int i = 0; i < n; ++i) {
          const int code = comm::ld_acquire_sys(rp + r0 + i);
          const uint8_t* from = reinterpret_cast<const uint8_t*>(ep.src[code >> 24]) + (long long)((code & 0xffffff) / ep.src_div) * row_bytes;
          bulk_load(base + slot * HALF + i * row_bytes, from, row_bytes, bar0 + 8u * slot);
        }
      };
      bool ok = true;
      if (nb > 0) issue(0);
      for (int b = 0; b < nb && ok; ++b) {
        if (b + 1 < nb) {
          if (b >= 1) bulk_wait_read();  // the store that last used the other slot has read it
          issue(b + 1);
        }
        const int slot = b & 1, r0 = b * rps, n = min(rps, nv - r0);
        if (!mbar_wait(bar0 + 8u * slot, uses[slot] & 1u, abort_flag)) { ok = false; break; }
        ++uses[slot];
        bulk_store(a_local + ((long long)mt * 128 + r0) * row_bytes, base + slot * HALF, (uint32_t)n * row_bytes);
        bulk_commit();
      }
      bulk_wait_all();
      fence_async_global();
      __threadfence();
      if (!ok) {
        atomicMax(status, ERR_GG_GATHER);
        s_ok = 0;
      }
    }
    __syncthreads();
    if (!s_ok) return;
    if (threadIdx.x == 0) st_release_gpu(&ep.tile_flags[mt], ep.epoch);
  }
}

struct Work {
  int m0, n0;       // output tile origin (rows mode: sorted row / output column; wgrad: dW row / dW column)
  int expert;       // -1: nothing to do
  int kb_begin, kb_end;  // K blocks (wgrad: blocks of 64 sorted rows)
};

template <int MODE>
__device__ __forceinline__ Work get_work(int t, const GroupedParams& g, int tiles_m, int tiles_n, int num_kb) {
  Work w;
  if (MODE == MODE_ROWS) {
    const int mt = t / tiles_n;
    w.m0 = mt * BM;
    w.n0 = (t % tiles_n) * BN;
    w.expert = g.tile_expert[mt];
    w.kb_begin = 0;
    w.kb_end = num_kb;
  } else {
    const int per_e = tiles_m * tiles_n;
    w.expert = t / per_e;
    const int r = t % per_e;
    w.m0 = (r / tiles_n) * BM;
    w.n0 = (r % tiles_n) * BN;
    w.kb_begin = g.offsets[w.expert] / BK;
    w.kb_end = g.offsets[w.expert + 1] / BK;
  }
  return w;
}

// MODE_ROWS : A = X sorted [R, K] K-major; B = stacked weights (B_K: [rows, K] K-major; else [rows = contraction, N] MN-major)
// MODE_WGRAD: A = dY sorted [R, N] MN-major (M = N features), B = X sorted [R, K] MN-major; D = dW_e
template <int MODE, bool B_K>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ Dv,
                    int M, int N, int K, long long ldd, GroupedParams g, int out_f32, int accumulate, int* __restrict__ status,
                    const EpRows ep, uint8_t* __restrict__ a_local) {
  const bool gather = MODE == MODE_ROWS && ep.src[0] != nullptr;
  const bool scatter = MODE == MODE_ROWS && ep.dst[0] != nullptr;
  const int n_copy = gather ? ep.n_copy_ctas : 0;
  if ((int)blockIdx.x < n_copy) {
    ep_gather(ep, (int)blockIdx.x, n_copy, M, K, a_local, g.tile_expert, status);
    return;
  }
  const int cta = (int)blockIdx.x - n_copy, n_ctas = (int)gridDim.x - n_copy;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + STAGES * STAGE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = (MODE == MODE_ROWS ? tiles_m : g.E * tiles_m) * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int landed = -1;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        const Work w = get_work<MODE>(t, g, tiles_m, tiles_n, num_kb);
        if (w.expert < 0) continue;
        const int brow = w.expert * g.b_rows_per_expert + g.b_row_offset;
        if (gather && landed != w.m0) {  // the copy CTAs must have brought this tile's rows
          const unsigned long long t0 = comm::now_ns();
          while (cpx::ld_acquire_gpu(&ep.tile_flags[w.m0 / BM]) < ep.epoch) {
            if (*abort_flag || comm::now_ns() - t0 > ep.timeout_ns) { ok = false; break; }
            __nanosleep(100);
          }
          if (!ok) { atomicMax(status, ERR_GG_TILE_WAIT); break; }
          cpx::fence_async_global();
          landed = w.m0;
        }
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (MODE == MODE_ROWS) {
            tma_load_2d(sa, &map_a, full_bar(stage), kb * BK, w.m0);
            if (B_K) {
              tma_load_2d(sb, &map_b, full_bar(stage), kb * BK, brow + w.n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &map_b, full_bar(stage), w.n0 + 64 * j, brow + kb * BK);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &map_a, full_bar(stage), w.m0 + 64 * j, kb * BK);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &map_b, full_bar(stage), w.n0 + 64 * j, kb * BK);
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_GG_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr bool A_MN = (MODE == MODE_WGRAD), B_MN = (MODE == MODE_WGRAD) || !B_K;
      constexpr uint32_t idesc = idesc_bf16(BM, BN, A_MN, B_MN);
      const uint32_t a_lo0 = desc_lo(base, !A_MN, BK * 128), b_lo0 = desc_lo(base + A_BYTES, !B_MN, BK * 128);
      constexpr int A_STEP = A_MN ? 128 : 2, B_STEP = B_MN ? 128 : 2;
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        const Work w = get_work<MODE>(t, g, tiles_m, tiles_n, num_kb);
        if (w.expert < 0) continue;
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), ((it >> 1) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_lo(d_tmem, a_lo + A_STEP * k, b_lo + B_STEP * k, idesc, ((kb - w.kb_begin) | k) ? 1u : 0u);
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) tc_commit(tfull_bar(buf));
        ++it;
      }
      if (!ok) {
        atomicMax(status, ERR_GG_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_ctas) {
      const Work w = get_work<MODE>(t, g, tiles_m, tiles_n, num_kb);
      if (w.expert < 0) continue;
      const int buf = it & 1;
      const bool empty = (w.kb_end <= w.kb_begin);  // wgrad of an expert that received no token
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after();
      int row = w.m0 + quarter * 32 + lane;
      uint8_t* dbase = reinterpret_cast<uint8_t*>(Dv) + (MODE == MODE_WGRAD ? (long long)w.expert * g.d_expert_stride * (out_f32 ? 4 : 2) : 0);
      bool live = row < M;
      if (scatter) {  // the row goes to the rank that owns its token; padding rows go nowhere
        const int code = live ? ep.row_peer[row] : -1;
        live = code >= 0;
        dbase = live ? reinterpret_cast<uint8_t*>(ep.dst[code >> 24]) : nullptr;
        row = code & 0xffffff;
      }
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld32(taddr0 + c * 32, r);
        tc_wait_ld();
        const int col = w.n0 + c * 32;
        if (live && col < N && !(empty && accumulate)) {
          if (out_f32) {
            float* d = reinterpret_cast<float*>(dbase) + (long long)row * ldd + col;
            for (int j = 0; j < 32 && col + j < N; ++j) {
              const float v = empty ? 0.f : __uint_as_float(r[j]);
              d[j] = accumulate ? d[j] + v : v;
            }
          } else {
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dbase) + (long long)row * ldd + col;
            if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(d) & 15) == 0) && !accumulate) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 pk;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const __nv_bfloat162 h = __floats2bfloat162_rn(empty ? 0.f : __uint_as_float(r[8 * j + 2 * q]),
                                                                 empty ? 0.f : __uint_as_float(r[8 * j + 2 * q + 1]));
                  pw[q] = *reinterpret_cast<const uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(d)[j] = pk;
              }
            } else {
              for (int j = 0; j < 32 && col + j < N; ++j) {
                float v = empty ? 0.f : __uint_as_float(r[j]);
                if (accumulate) v += __bfloat162float(d[j]);
                d[j] = __float2bfloat16_rn(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
      ++it;
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR_GG_EPILOGUE);
      *abort_flag = 1;
    }
    if (scatter) __threadfence_system();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (scatter && threadIdx.x == 0 && *abort_flag == 0) {
    // the last CTA tells every rank that all of this rank's output rows are in place
    const int done = atomicAdd(ep.done_counter, 1);
    if (done == (int)gridDim.x - 1) {
      *ep.done_counter = 0;
      __threadfence_system();
      for (int p = 0; p < ep.world; ++p)
        comm::st_release_sys(cpx::flag_slot(ep.flags[p], KIND_EP, ep.rank, ep.signal_unit, ep.max_units), ep.epoch);
    }
  }
}

template <int MODE, bool B_K>
int launch_gg(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd, const GroupedParams& g,
              bool out_f32, bool accumulate, int* status, cudaStream_t st, const EpRows& ep = EpRows(), void* a_local = nullptr) {
  auto kern = gemm_grouped_kernel<MODE, B_K>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = (MODE == MODE_ROWS ? 1 : g.E) * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int n_copy = (MODE == MODE_ROWS && ep.src[0] != nullptr) ? ep.n_copy_ctas : 0;
  int gemm_ctas = sms - n_copy;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  kern<<<gemm_ctas + n_copy, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, D, M, N, K, ldd, g, out_f32 ? 1 : 0, accumulate ? 1 : 0, status,
                                                            ep, (uint8_t*)a_local);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

// Y[R, N] = X[R, K] . op(W_e): rows mode.  `w_rows` / `w_cols` describe the 2-D view of the stacked weight buffer.
int gemm_grouped_rows(const void* X, const void* W, void* Y, int R, int N, int K, long long ldx, long long w_rows, long long w_cols,
                      long long ldy, bool w_kmajor, const GroupedParams& g, int* status, cudaStream_t st, const EpRows* ep_in) {
  if (R <= 0 || N <= 0 || K <= 0) return 0;
  if (R % BM) return -2;
  if (!w_kmajor && (K % BK)) return -3;  // MN-major weight: contraction rows of one expert must be whole K blocks
  EpRows ep;
  if (ep_in != nullptr && ep_in->world > 1) {
    ep = *ep_in;
    if (ep.world > 8 || ep.rank < 0 || ep.rank >= ep.world || ep.row_peer == nullptr) return -6;
    if (ep.src[0] != nullptr) {  // rows are whole 16-byte multiples, one slot holds at least one row, dense sorted buffer
      if (ep.n_copy_ctas < 1 || ep.n_copy_ctas > 64 || ep.tile_flags == nullptr || ep.src_div < 1) return -6;
      if (K % 8 || K * 2 > STAGES * STAGE_BYTES / 2 || ldx != K) return -7;
    }
    if (ep.dst[0] != nullptr && (ep.done_counter == nullptr || N % 32 || ldy % 8)) return -7;
  }
  CUtensorMap ma, mb;
  if (!cache().get(&ma, X, K, R, ldx, BK, BM)) return -1000 - g_last_map_error;
  const bool okb = w_kmajor ? cache().get(&mb, W, w_cols, w_rows, w_cols, BK, BN) : cache().get(&mb, W, w_cols, w_rows, w_cols, 64, BK);
  if (!okb) return -2000 - g_last_map_error;
  return w_kmajor ? launch_gg<MODE_ROWS, true>(ma, mb, Y, R, N, K, ldy, g, false, false, status, st, ep, const_cast<void*>(X))
                  : launch_gg<MODE_ROWS, false>(ma, mb, Y, R, N, K, ldy, g, false, false, status, st, ep, const_cast<void*>(X));
}

// dW_e[N, K] (+)= dY_e^T X_e for every expert; D is the stacked gradient buffer (row stride ldd, expert stride in g).
int gemm_grouped_wgrad(const void* dY, const void* X, void* D, int R, int N, int K, long long lddy, long long ldx, long long ldd,
                       bool out_f32, bool accumulate, const GroupedParams& g, int* status, cudaStream_t st) {
  if (R <= 0 || N <= 0 || K <= 0 || g.E <= 0) return 0;
  if (R % BM) return -2;
  CUtensorMap ma, mb;
  if (!cache().get(&ma, dY, N, R, lddy, 64, BK)) return -1000 - g_last_map_error;
  if (!cache().get(&mb, X, K, R, ldx, 64, BK)) return -2000 - g_last_map_error;
  return launch_gg<MODE_WGRAD, true>(ma, mb, D, N, K, /*K loop from offsets*/ 0, ldd, g, out_f32, accumulate, status, st);
}

}  // namespace ab
