// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a, tcgen05 + TMA + TMEM).
//
//   gemm_allgather   (column-parallel linear, sequence-sharded input):  Y[M, N] = concat_r(X_r)[M, K] * W[N, K]^T
//       Every rank keeps X in a symmetric buffer X_full[M, K] and owns row block r = rank.  ONE persistent kernel:
//       a few "copy CTAs" announce "my block is ready", wait (bounded) for each peer's announcement and pull the
//       peers' row blocks over NVLink into the local X_full (16-byte coherent loads, each remote byte crosses the link
//       exactly once), publishing one flag per block; the remaining CTAs run the tcgen05 GEMM, starting with the
//       tiles of the local block and taking remote blocks in arrival order - their TMA producer polls the block flag
//       (bounded) before it loads from LOCAL memory.  The transfer of block i+1 overlaps the MMAs of block i.
//   gemm_reducescatter (row-parallel linear):  Y_r[M/W, N] = sum_p (X_p[M, K_p] * W_p[N, K_p]^T)[rows of r]
//       ONE persistent kernel: output tiles are computed remote-destination first and the epilogue stores each tile
//       straight into the destination rank's staging slot [source rank][M/W, N] (bf16, plain peer stores: no atomics,
//       fixed summation order); a per-destination counter lets the last epilogue warp publish "all my tiles for you
//       are there"; when a CTA runs out of tiles its epilogue warps wait (bounded) for every peer's flag and reduce
//       the W staged partials of the local row block in fp32.
// Both replace "NCCL collective + cuBLAS GEMM" pairs; the reference has no tensor parallelism at all
// (scripts/tools/train.py:513-519 parses --tp_size and drops it).  No TMA multicast is used; TMA only ever reads
// this GPU's own memory.  Every wait is bounded by a globaltimer budget; expiry records a code in `status`.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"
#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

using namespace tc;
using namespace tmah;
using namespace comm;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
enum : int { MODE_AG = 1, MODE_RS = 2 };
enum : int { ERR_TP_PRODUCER = 51, ERR_TP_MMA = 52, ERR_TP_EPILOGUE = 53, ERR_TP_COPY = 54, ERR_TP_REDUCE = 55 };
constexpr int KIND_AG = 2, KIND_RS = 3;  // flag planes (astrai_b200/parallel/symm.py)

__device__ __forceinline__ int* flag_slot(void* base, int kind, int src, int unit, int max_units) {
  return reinterpret_cast<int*>(base) + ((long long)kind * MAX_RANKS + src) * max_units + unit;
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

// Tile t of the schedule -> (m0, n0).  Row blocks are visited starting at `first_block` (the local block for the
// all-gather, the first remote destination for the reduce-scatter); inside a block column tiles vary fastest.
struct TileCoord { int m0, n0, block; };
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m_per_block, int tiles_n, int world, int first_block) {
  const int per_block = tiles_m_per_block * tiles_n;
  const int bi = t / per_block, r = t % per_block;
  const int block = (first_block + bi) % world;
  return {(block * tiles_m_per_block + r / tiles_n) * BM, (r % tiles_n) * BN, block};
}

template <int MODE, bool B_K>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 __nv_bfloat16* __restrict__ D, int M, int N, int K, long long ldd, TpGemmParams p, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Ms = M / p.world;  // rows per block (multiple of BM)
  const int tiles_m_blk = Ms / BM, tiles_n = (N + BN - 1) / BN, num_tiles = tiles_m_blk * p.world * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int n_copy = (MODE == MODE_AG) ? p.n_copy_ctas : 0;

  if (MODE == MODE_AG && (int)blockIdx.x < n_copy) {
    // ------------------------------------------------------------ copy CTAs: pull the peers' row blocks into X_full
    __shared__ int s_ok;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(flag_slot(p.flags[threadIdx.x], KIND_AG, p.rank, p.unit, p.max_units), p.epoch);
    }
    const long long vec_per_block = (long long)Ms * K / 8;  // 16-byte vectors in one row block
    for (int i = 1; i < p.world; ++i) {
      const int src = (p.rank + i) % p.world;
      if (threadIdx.x == 0) {
        s_ok = wait_flag(flag_slot(p.flags[p.rank], KIND_AG, src, p.unit, p.max_units), p.epoch, p.timeout_ns) ? 1 : 0;
        if (!s_ok) atomicMax(status, ERR_TP_COPY);
      }
      __syncthreads();
      if (!s_ok) return;  // the GEMM CTAs time out on the block flag and report as well
      const uint4* from = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.x_full[src]) + (long long)src * Ms * K);
      uint4* to = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.x_full[p.rank]) + (long long)src * Ms * K);
      constexpr int U = 4;
      const long long stride = (long long)n_copy * NUM_THREADS;
      for (long long v0 = (long long)blockIdx.x * NUM_THREADS + threadIdx.x; v0 < vec_per_block; v0 += stride * U) {
        uint4 tmp[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (v0 + u * stride < vec_per_block) tmp[u] = ld_sys_u4(from + v0 + u * stride);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (v0 + u * stride < vec_per_block) to[v0 + u * stride] = tmp[u];
      }
      fence_async_global();  // the GEMM CTAs read these rows through TMA (async proxy)
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int done = atomicAdd(&p.chunk_counter[src], 1);
        if (done == n_copy - 1) {
          p.chunk_counter[src] = 0;
          st_release_gpu(&p.chunk_flags[src], p.epoch);
        }
      }
    }
    return;
  }

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
  const int cta = (int)blockIdx.x - n_copy, n_ctas = (int)gridDim.x - n_copy;
  const int first_block = (MODE == MODE_RS) ? (p.rank + 1) % p.world : p.rank;

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
      int stage = 0, ready_block = -1;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        const TileCoord tcd = tile_coord(t, tiles_m_blk, tiles_n, p.world, first_block);
        if (MODE == MODE_AG && tcd.block != p.rank && tcd.block != ready_block) {
          // rows of a remote block: wait until the copy CTAs have landed it in local memory
          const unsigned long long t0 = now_ns();
          while (ld_acquire_gpu(&p.chunk_flags[tcd.block]) < p.epoch) {
            if (*abort_flag || now_ns() - t0 > p.timeout_ns) {
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_async_global();
          ready_block = tcd.block;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &map_a, full_bar(stage), kb * BK, tcd.m0);
          if (B_K) {
            tma_load_2d(sb, &map_b, full_bar(stage), kb * BK, tcd.n0);
          } else {  // B stored [K, N]: 64-column boxes, one per 64 output columns
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &map_b, full_bar(stage), tcd.n0 + 64 * j, kb * BK);
          }
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_TP_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BM, BN, false, !B_K);
      const uint32_t a_lo0 = desc_lo(base, true, 0), b_lo0 = desc_lo(base + A_BYTES, B_K, BK * 128);
      constexpr int B_STEP = B_K ? 2 : 128;  // K-major: 32 B per 16-wide K slice; MN-major: 16 rows of 128 B
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas, ++it) {
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
          const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) tc_mma_lo(d_tmem, a_lo + 2 * k, b_lo + B_STEP * k, idesc, (kb | k) ? 1u : 0u);
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
      if (!ok) {
        atomicMax(status, ERR_TP_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_ctas, ++it) {
      const int buf = it & 1;
      const TileCoord tcd = tile_coord(t, tiles_m_blk, tiles_n, p.world, first_block);
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tcd.m0 + quarter * 32 + lane;
      __nv_bfloat16* drow;
      if (MODE == MODE_RS) {
        // rows of block `dst` go to rank dst's staging slot of this source rank
        __nv_bfloat16* stage_dst = reinterpret_cast<__nv_bfloat16*>(p.stage[tcd.block]);
        drow = stage_dst + ((long long)p.rank * Ms + (row - tcd.block * Ms)) * N;
      } else {
        drow = D + (long long)row * ldd;
      }
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld32(taddr0 + c * 32, r);
        tc_wait_ld();
        const int col = tcd.n0 + c * 32;
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
      if (MODE == MODE_RS) __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(tempty_bar(buf));
        if (MODE == MODE_RS) {
          // count warp arrivals per destination; the last one publishes the flag on the destination rank
          const int done = atomicAdd(&p.tile_counter[tcd.block], 1);
          if (done == 4 * tiles_m_blk * tiles_n - 1) {
            __threadfence_system();
            st_release_sys(flag_slot(p.flags[tcd.block], KIND_RS, p.rank, p.unit, p.max_units), p.epoch);
          }
        }
      }
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR_TP_EPILOGUE);
      *abort_flag = 1;
    }
    if (MODE == MODE_RS && ok && p.fuse_reduce) {
      // ---- reduce phase: every peer's partial rows of the local block have to be in the staging buffer
      bool got = true;
      if (lane < p.world) got = wait_flag(flag_slot(p.flags[p.rank], KIND_RS, lane, p.unit, p.max_units), p.epoch, p.timeout_ns);
      got = __all_sync(0xffffffffu, got);
      if (!got) {
        if (lane == 0) atomicMax(status, ERR_TP_REDUCE);
      } else {
        const __nv_bfloat16* st = reinterpret_cast<const __nv_bfloat16*>(p.stage[p.rank]);
        const long long n_vec = (long long)Ms * N / 8, slot = (long long)Ms * N;
        const long long tid = (long long)cta * 128 + (warp - 2) * 32 + lane, nthr = (long long)n_ctas * 128;
        for (long long v = tid; v < n_vec; v += nthr) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int s = 0; s < p.world; ++s) {
            const uint4 raw = ld_sys_u4(st + s * slot + v * 8);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = __bfloat1622float2(h[q]);
              acc[2 * q] += f.x, acc[2 * q + 1] += f.y;
            }
          }
          uint4 pk;
          uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
            pw[q] = *reinterpret_cast<const uint32_t*>(&h);
          }
          reinterpret_cast<uint4*>(p.rs_out)[v] = pk;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Stand-alone reduce of the staged partials (used when the fused phase is switched off, e.g. when several ranks are
// emulated on one GPU and their kernels must not wait for one another).
__global__ void tp_reduce_kernel(const __nv_bfloat16* __restrict__ st, __nv_bfloat16* __restrict__ out, long long n_vec,
                                 long long slot, int world) {
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s) {
      const uint4 raw = *reinterpret_cast<const uint4*>(st + s * slot + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += f.x, acc[2 * q + 1] += f.y;
      }
    }
    uint4 pk;
    uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      pw[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(out)[v] = pk;
  }
}

template <int MODE, bool B_K>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* D, int M, int N, int K, long long ldd, const TpGemmParams& p,
           int* status, cudaStream_t st) {
  auto kern = gemm_comm_kernel<MODE, B_K>;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  // every CTA must be resident at once: copy CTAs and GEMM CTAs wait on one another's flags
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  int gemm_ctas = sms - (MODE == MODE_AG ? p.n_copy_ctas : 0);
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  const int grid = gemm_ctas + (MODE == MODE_AG ? p.n_copy_ctas : 0);
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, (__nv_bfloat16*)D, M, N, K, ldd, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int check(const TpGemmParams& p, int M, int N, int K) {
  if (p.world < 1 || p.world > MAX_RANKS || p.rank < 0 || p.rank >= p.world) return -1;
  if (M % (p.world * BM) || N % 32 || K % 8) return -2;  // row blocks are whole tiles; 32-column epilogue chunks
  if (p.unit < 0 || p.unit >= p.max_units) return -3;
  return 0;
}

}  // namespace

int gemm_allgather(const void* W, bool w_kmajor, void* Y, int M, int N, int K, long long ldy, const TpGemmParams& p,
                   int* status, cudaStream_t st) {
  if (int rc = check(p, M, N, K)) return rc;
  if (p.n_copy_ctas < 1 || p.n_copy_ctas > 64) return -6;
  CUtensorMap ma, mb;
  if (!cache().get(&ma, p.x_full[p.rank], K, M, K, BK, BM)) return -1000 - g_last_map_error;
  const bool okb = w_kmajor ? cache().get(&mb, W, K, N, K, BK, BN) : cache().get(&mb, W, N, K, N, 64, BK);
  if (!okb) return -2000 - g_last_map_error;
  return w_kmajor ? launch<MODE_AG, true>(ma, mb, Y, M, N, K, ldy, p, status, st)
                  : launch<MODE_AG, false>(ma, mb, Y, M, N, K, ldy, p, status, st);
}

int gemm_reducescatter(const void* X, const void* W, bool w_kmajor, int M, int N, int K, const TpGemmParams& p,
                       int* status, cudaStream_t st) {
  if (int rc = check(p, M, N, K)) return rc;
  CUtensorMap ma, mb;
  if (!cache().get(&ma, X, K, M, K, BK, BM)) return -1000 - g_last_map_error;
  const bool okb = w_kmajor ? cache().get(&mb, W, K, N, K, BK, BN) : cache().get(&mb, W, N, K, N, 64, BK);
  if (!okb) return -2000 - g_last_map_error;
  if (cudaMemsetAsync(p.tile_counter, 0, sizeof(int) * MAX_RANKS, st) != cudaSuccess) return -7;
  return w_kmajor ? launch<MODE_RS, true>(ma, mb, nullptr, M, N, K, N, p, status, st)
                  : launch<MODE_RS, false>(ma, mb, nullptr, M, N, K, N, p, status, st);
}

int tp_reduce(const void* stage, void* out, long long rows, int N, int world, cudaStream_t st) {
  const long long n_vec = rows * N / 8;
  if (n_vec == 0) return 0;
  long long g = (n_vec + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  tp_reduce_kernel<<<(int)g, 256, 0, st>>>((const __nv_bfloat16*)stage, (__nv_bfloat16*)out, n_vec, rows * N, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
