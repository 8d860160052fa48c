// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): one 256x256 output tile per pair of SMs.
//
// Why pairs: with one CTA per 128x256 tile every CTA pulls 48 KB of operands per 64-wide K block, about 85 FLOP per
// byte of L2->shared traffic, and the kernel saturates L2 before the tensor cores.  In a pair each CTA loads only its
// own 128 rows of A and HALF of the B tile (128 of the 256 rows); the 2-CTA MMA reads the other half from the peer's
// shared memory.  That is 32 KB per CTA per K block (170 FLOP/byte) and leaves room for a 6-stage ring.
// No TMA multicast is used anywhere: each CTA issues plain loads for its own halves.
//
// Roles per CTA (6 warps): warp 0 TMA producer (both CTAs), warp 1 MMA issuer (leader CTA only; owns the TMEM
// allocation in both), warps 2..5 epilogue (both CTAs, each drains its own 128 accumulator rows).
// Barriers: `full` lives in the leader and counts the bytes of BOTH CTAs' loads; `empty` and `tmem_full` exist in both
// CTAs and are signalled by multicast tcgen05.commit; `tmem_empty` lives in the leader and collects one arrival per
// epilogue warp of both CTAs.  Every wait is bounded; see gemm_tcgen05.cu for the abort protocol.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

using namespace tc;
using namespace tmah;

constexpr int BM = 128;       // rows per CTA (pair tile: 256)
constexpr int BN = 256;       // columns of the pair tile
constexpr int BNH = BN / 2;   // B rows loaded by each CTA
constexpr int BK = 64, STAGES = 6, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KB
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

enum : int { ERR_PRODUCER = 11, ERR_MMA_FULL = 12, ERR_MMA_TMEM = 13, ERR_EPILOGUE = 14 };

__device__ __forceinline__ uint64_t make_desc2(uint32_t saddr, bool kmajor) {
  const uint64_t lbo = kmajor ? 1ull : (uint64_t)((BK * 128) >> 4);
  const uint64_t sbo = 1024 >> 4;
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

struct TileCoord { int m0, n0; };
__device__ __forceinline__ TileCoord tile_coord2(int t, int tiles_m, int tiles_n) {
  constexpr int G = 8;  // 8 pair-rows (2048 output rows) sweep all column tiles
  const int per_group = G * tiles_n;
  const int g = t / per_group, r = t % per_group;
  const int rows = min(G, tiles_m - g * G);
  return {(g * G + r % rows) * (2 * BM), (r / rows) * BN};
}

// Work list of one CTA pair.  Full rounds: tile p + r * P of the rasterised order, 256 columns wide.  The tiles left
// over after the last full round (fewer than P) would keep most pairs idle for a whole tile time; when twice their
// number still fits into one round they are cut into two 128-column halves, one per pair, so the tail costs about
// half a tile time instead of one.
struct Work {
  int t, n_off, bn;
};
struct Schedule {
  int num_tiles, P, p, full_rounds, rem;
  bool split;
  __device__ Schedule(int num_tiles_, int P_, int p_) : num_tiles(num_tiles_), P(P_), p(p_) {
    full_rounds = num_tiles / P;
    rem = num_tiles - full_rounds * P;
    split = rem > 0 && 2 * rem <= P;
  }
  __device__ bool get(int i, Work& w) const {
    if (i < full_rounds) {
      w = {p + i * P, 0, BN};
      return true;
    }
    if (i > full_rounds) return false;
    if (split) {
      if (p >= 2 * rem) return false;
      w = {full_rounds * P + (p >> 1), (p & 1) * (BN / 2), BN / 2};
      return true;
    }
    if (p >= rem) return false;
    w = {full_rounds * P + p, 0, BN};
    return true;
  }
};

template <bool A_K, bool B_K, bool OUT_F32, bool ACCUM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ Dv,
             int M, int N, int K, long long ldd, int* __restrict__ status) {
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
  volatile int* never_flag = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN, num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // leader's copy is the one in use
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);  // 4 epilogue warps x 2 CTAs arrive on the leader's copy
    }
    *abort_flag = 0;
    *never_flag = 0;
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
  cluster_sync();  // both CTAs' barriers are initialised before anybody signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const Schedule sched(num_tiles, num_pairs, pair);
      Work wk;
      for (int wi = 0; ok && sched.get(wi, wk); ++wi) {
        const TileCoord tc = tile_coord2(wk.t, tiles_m, tiles_n);
        const bool half = wk.bn != BN;  // each CTA then supplies 64 rows of B instead of 128
        const int m0 = tc.m0 + (int)rank * BM, n0 = tc.n0 + wk.n_off + (int)rank * (wk.bn / 2);
        // K-major B: the 128-row box is loaded either way (its first 64 rows are the half tile's); MN-major B: one
        // 64-column box instead of two
        const uint32_t stage_tx = (!B_K && half) ? (uint32_t)(A_BYTES + B_BYTES / 2) : (uint32_t)STAGE_BYTES;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint32_t fb = mapa(full_bar(stage), 0);  // byte counts go to the leader's barrier
          if (leader) mbar_expect_tx(full_bar(stage), 2 * stage_tx);
          const int k0 = kb * BK;
          if (A_K) {
            tma_load_2d_cg2(sa, &map_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_cg2(sa + j * (BK * 128), &map_a, fb, m0 + 64 * j, k0);
          }
          if (B_K) {
            tma_load_2d_cg2(sb, &map_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j)
              if (j == 0 || !half) tma_load_2d_cg2(sb + j * (BK * 128), &map_b, fb, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc_base = (1u << 4) | (1u << 7) | (1u << 10) | ((A_K ? 0u : 1u) << 15) |
                                      ((B_K ? 0u : 1u) << 16) | ((uint32_t)((2 * BM) >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      const Schedule sched(num_tiles, num_pairs, pair);
      Work wk;
      for (; ok && sched.get(it, wk); ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        const uint32_t idesc = idesc_base | ((uint32_t)(wk.bn >> 3) << 17);
        if (!mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag)) {
          atomicMax(status, ERR_MMA_TMEM);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            atomicMax(status, ERR_MMA_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t da = make_desc2(sa, A_K), db = make_desc2(sb, B_K);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ka = (uint64_t)((A_K ? k * UMMA_K * 2 : k * UMMA_K * 128) >> 4);
            const uint64_t kbo = (uint64_t)((B_K ? k * UMMA_K * 2 : k * UMMA_K * 128) >> 4);
            tc_mma_cg2(d_tmem, da + ka, db + kbo, idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit_cg2(empty_bar(stage), 3);  // frees the slot in both CTAs
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) tc_commit_cg2(tfull_bar(buf), 3);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    const uint32_t tempty_leader0 = mapa(tempty_bar(0), 0), tempty_leader1 = mapa(tempty_bar(1), 0);
    int it = 0;
    bool ok = true;
    const Schedule sched(num_tiles, num_pairs, pair);
    Work wk;
    for (; ok && sched.get(it, wk); ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      TileCoord tc = tile_coord2(wk.t, tiles_m, tiles_n);
      tc.n0 += wk.n_off;
      if (!mbar_wait(tfull_bar(buf), acc_phase, abort_flag)) {
        if (lane == 0) atomicMax(status, ERR_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tc.m0 + (int)rank * BM + quarter * 32 + lane;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < wk.bn / 32; ++c) {
        uint32_t r[32];
        tc_ld32(taddr0 + c * 32, r);
        tc_wait_ld();
        const int col = tc.n0 + c * 32;
        if (row < M && col < N) {
          if (OUT_F32) {
            float* d = reinterpret_cast<float*>(Dv) + (long long)row * ldd + col;
            const bool vec = (col + 32 <= N) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (ACCUM) {
                  const float4 o = reinterpret_cast<float4*>(d)[j];
                  v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
                }
                reinterpret_cast<float4*>(d)[j] = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < N; ++j) d[j] = __uint_as_float(r[j]) + (ACCUM ? d[j] : 0.f);
            }
          } else {
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(Dv) + (long long)row * ldd + col;
            const bool vec = (col + 32 <= N) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 pk;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
                uint4 old;
                if (ACCUM) old = reinterpret_cast<uint4*>(d)[j];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float lo = __uint_as_float(r[8 * j + 2 * q]), hi = __uint_as_float(r[8 * j + 2 * q + 1]);
                  if (ACCUM) {
                    const float2 o = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&old)[q]);
                    lo += o.x, hi += o.y;
                  }
                  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                  pw[q] = *reinterpret_cast<const uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(d)[j] = pk;
              }
            } else {
              for (int j = 0; j < 32 && col + j < N; ++j) {
                float f = __uint_as_float(r[j]);
                if (ACCUM) f += __bfloat162float(d[j]);
                d[j] = __float2bfloat16_rn(f);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? tempty_leader1 : tempty_leader0);
    }
    if (!ok && lane == 0) *abort_flag = 1;
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // neither CTA leaves (or frees TMEM) while its peer may still read its shared memory or signal it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

template <bool A_K, bool B_K, bool OUT_F32, bool ACCUM>
int launch2(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd, int* status,
            cudaStream_t st) {
  auto kern = gemm2_kernel<A_K, B_K, OUT_F32, ACCUM>;
  static bool configured = false;
  static int max_pairs = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sms / 2;
    }
    max_pairs = clusters < sms / 2 ? clusters : sms / 2;
    configured = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, D, M, N, K, ldd, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int gemm_bf16_2cta(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                   long long ldd, bool a_kmajor, bool b_kmajor, bool out_f32, bool accumulate, int* status,
                   cudaStream_t st) {
  CUtensorMap ma, mb;
  const bool oka = a_kmajor ? cache().get(&ma, A, K, M, lda, BK, BM) : cache().get(&ma, A, M, K, lda, 64, BK);
  if (!oka) return -1000 - g_last_map_error;
  const bool okb = b_kmajor ? cache().get(&mb, B, K, N, ldb, BK, BNH) : cache().get(&mb, B, N, K, ldb, 64, BK);
  if (!okb) return -2000 - g_last_map_error;
  const int sel = (a_kmajor ? 8 : 0) | (b_kmajor ? 4 : 0) | (out_f32 ? 2 : 0) | (accumulate ? 1 : 0);
  switch (sel) {
#define AB_CASE(i, a, b, f, c) \
  case i: return launch2<a, b, f, c>(ma, mb, D, M, N, K, ldd, status, st);
    AB_CASE(0, false, false, false, false) AB_CASE(1, false, false, false, true)
    AB_CASE(2, false, false, true, false) AB_CASE(3, false, false, true, true)
    AB_CASE(4, false, true, false, false) AB_CASE(5, false, true, false, true)
    AB_CASE(6, false, true, true, false) AB_CASE(7, false, true, true, true)
    AB_CASE(8, true, false, false, false) AB_CASE(9, true, false, false, true)
    AB_CASE(10, true, false, true, false) AB_CASE(11, true, false, true, true)
    AB_CASE(12, true, true, false, false) AB_CASE(13, true, true, false, true)
    AB_CASE(14, true, true, true, false) AB_CASE(15, true, true, true, true)
#undef AB_CASE
  }
  return -3;
}

}  // namespace ab
