// bf16 GEMM on the 5th-generation tensor cores (sm_100a): D[M,N] (+)= A x B, fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 0      : TMA producer   - cp.async.bulk.tensor (no multicast) into a 4-stage ring of 128B-swizzled tiles
//   warp 1      : MMA issuer     - one lane issues tcgen05.mma (M128 x N256 x K16) per 16-wide K slice; owns TMEM
//   warps 2..5  : epilogue       - tcgen05.ld the finished 128x256 fp32 accumulator, cast / accumulate, store
// The accumulator is double-buffered in TMEM (2 x 256 columns) so the epilogue of tile i overlaps the MMAs of
// tile i+1.  Both operands may be K-major or MN-major (the transposes needed by dgrad / wgrad are expressed in
// the shared-memory descriptors, never materialised).  Replaces cuBLAS behind F.linear of the reference
// (astrai/model/components/linear.py:24) for forward, dgrad and wgrad.
//
// Every wait on an mbarrier is bounded (about two seconds of globaltimer); on expiry the kernel records a code
// in `status`, drains the copies it still has in flight, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdlib.h>

#include <map>
#include <mutex>
#include <tuple>

#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

enum : int { ERR_PRODUCER = 1, ERR_MMA_FULL = 2, ERR_MMA_TMEM = 3, ERR_EPILOGUE = 4 };

using namespace tc;
using namespace tmah;

// Shared-memory matrix descriptor for a 128-byte-swizzled tile (version 1, base offset 0).
//   K-major : rows of 64 bf16 (128 B); 8-row groups 1024 B apart (SBO); LBO unused (1).
//   MN-major: rows of 64 MN-elements (128 B) per K index; 8-K groups 1024 B apart (SBO);
//             the next block of 64 MN-elements starts BK*128 B later (LBO).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, bool kmajor) {
  const uint64_t lbo = kmajor ? 1ull : (uint64_t)((BK * 128) >> 4);
  const uint64_t sbo = 1024 >> 4;
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

struct TileCoord { int m0, n0; };
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n) {
  // groups of 16 row-tiles sweep all column-tiles: keeps a wave's A and B footprints in L2
  constexpr int G = 16;
  const int per_group = G * tiles_n;
  const int g = t / per_group, r = t % per_group;
  const int rows = min(G, tiles_m - g * G);
  return {(g * G + r % rows) * BM, (r / rows) * BN};
}

template <bool A_K, bool B_K, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ Dv,
            int M, int N, int K, long long ldd, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + STAGES * STAGE_BYTES);
  // bars: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty, then tmem ptr + abort flag
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* never_flag = reinterpret_cast<volatile int*>(tmem_holder + 2);  // stays 0: time limit only

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, num_tiles = tiles_m * tiles_n;
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
    *never_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_K) {
            tma_load_2d(sa, &map_a, full_bar(stage), k0, tc.m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &map_a, full_bar(stage), tc.m0 + 64 * j, k0);
          }
          if (B_K) {
            tma_load_2d(sb, &map_b, full_bar(stage), k0, tc.n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &map_b, full_bar(stage), tc.n0 + 64 * j, k0);
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_PRODUCER);
        *abort_flag = 1;
        // Drain: every stage issued in the previous lap either completed or gets a bounded wait here, so no
        // bulk copy is still writing this CTA's shared memory when it exits.
        for (int s = 0; s < STAGES; ++s) {
          const uint32_t ph = (s < stage) ? phase : (phase ^ 1u);
          (void)mbar_wait(full_bar(s), ph, never_flag);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_K ? 0u : 1u) << 15) |
                                 ((B_K ? 0u : 1u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
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
          const uint64_t da = make_desc(sa, A_K), db = make_desc(sb, B_K);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: +32 B per 16-wide K slice inside the swizzle atom; MN-major: +16 rows of 128 B
            const uint64_t ka = (uint64_t)((A_K ? k * UMMA_K * 2 : k * UMMA_K * 128) >> 4);
            const uint64_t kbo = (uint64_t)((B_K ? k * UMMA_K * 2 : k * UMMA_K * 128) >> 4);
            tc_mma(d_tmem, da + ka, db + kbo, idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) are the only ones this warp may read
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
      if (!mbar_wait(tfull_bar(buf), acc_phase, abort_flag)) {
        if (lane == 0) atomicMax(status, ERR_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tc.m0 + quarter * 32 + lane;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
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
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
    if (!ok && lane == 0) *abort_flag = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ------------------------------------------------------------------ host side
template <bool A_K, bool B_K, bool OUT_F32, bool ACCUM>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd, int* status,
           cudaStream_t st) {
  auto kern = gemm_kernel<A_K, B_K, OUT_F32, ACCUM>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, D, M, N, K, ldd, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
              bool a_kmajor, bool b_kmajor, bool out_f32, bool accumulate, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
    return -1;  // TMA needs 16-byte aligned bases and row strides
  static const bool force_single = [] {
    const char* e = getenv("ASTRAI_B200_GEMM_1CTA");
    return e && e[0] == '1';
  }();
  if (M >= 256 && !force_single)
    return gemm_bf16_2cta(A, B, D, M, N, K, lda, ldb, ldd, a_kmajor, b_kmajor, out_f32, accumulate, status, st);
  CUtensorMap ma, mb;
  // K-major operand: stored [rows=MN, cols=K]; box 64(K) x tile rows.  MN-major: stored [rows=K, cols=MN]; box 64(MN) x BK.
  const bool oka = a_kmajor ? cache().get(&ma, A, K, M, lda, BK, BM) : cache().get(&ma, A, M, K, lda, 64, BK);
  if (!oka) return -1000 - g_last_map_error;  // tensor map of A rejected: -1000 - CUresult
  const bool okb = b_kmajor ? cache().get(&mb, B, K, N, ldb, BK, BN) : cache().get(&mb, B, N, K, ldb, 64, BK);
  if (!okb) return -2000 - g_last_map_error;  // tensor map of B rejected: -2000 - CUresult
  const int sel = (a_kmajor ? 8 : 0) | (b_kmajor ? 4 : 0) | (out_f32 ? 2 : 0) | (accumulate ? 1 : 0);
  switch (sel) {
#define AB_CASE(i, a, b, f, c) \
  case i: return launch<a, b, f, c>(ma, mb, D, M, N, K, ldd, status, st);
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
