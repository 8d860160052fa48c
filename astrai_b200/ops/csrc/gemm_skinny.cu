// Skinny bf16 GEMM for decode-sized batches (M <= 256 tokens): Y[M, N] = X[M, K] . W[N, K]^T on tcgen05.
//
// With a handful of tokens the op is a stream over the weight matrix: what matters is that all 148 SMs pull bytes.
// The output-stationary 128 x 256 tiles of the training GEMM would give N / 256 CTAs (8 for the 1B model's down
// projection).  Here the operands are swapped and K is split:
//   * the WEIGHT is the M operand of the MMA (128 output features per CTA, K-major as stored), the tokens are the N
//     operand (padded to 16 / 32 / 64 / 128 / 256 by TMA zero fill), so a CTA's accumulator is Y^T[128 features, tokens] in TMEM;
//   * K is split across the CTAs of a thread-block cluster (1, 2, 4 or 8 CTAs per 128-feature tile, chosen so that
//     about 148..300 CTAs exist); each CTA runs a 4-stage TMA ring over its slice of K;
//   * the partial accumulators never touch global memory: every CTA parks its fp32 tile in its own shared memory, the
//     cluster synchronises, and each CTA sums one slice of the tile over all peers through distributed shared memory
//     (ld.shared::cluster) in a fixed order and writes bf16.
// No atomics, no workspace, one launch (CUDA-graph safe).  Replaces cuBLAS GEMV-like calls behind
// F.linear in the reference's decode path (astrai/model/components/linear.py:24).
// All mbarrier waits are bounded; expiry records a code in `status`.
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

constexpr int BF = 128;  // output features per CTA (MMA M)
constexpr int BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int W_BYTES = BF * BK * 2;  // 16 KB
constexpr int NUM_THREADS = 192;
enum : int { ERR_SK_PRODUCER = 71, ERR_SK_MMA = 72, ERR_SK_EPILOGUE = 73 };

template <int TOK>  // padded token count: 16, 32, 64, 128 or 256
struct SkCfg {
  static constexpr int X_BYTES = TOK * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int RED_BYTES = TOK * BF * 4;  // parked fp32 tile [token][feature]; reuses the ring after the MMAs
  static_assert(RED_BYTES <= STAGES * STAGE_BYTES, "the parked tile must fit in the ring");
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}

template <int TOK>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   __nv_bfloat16* __restrict__ Y, int M, int N, int K, long long ldy, int kb_per_split, int* __restrict__ status) {
  using C = SkCfg<TOK>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + STAGES * C::STAGE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t done_bar = bar0 + 8u * (2 * STAGES);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cs = (int)cluster_nctarank(), split = (int)cluster_ctarank();
  const int n0 = ((int)blockIdx.x / cs) * BF;
  const int num_kb = (K + BK - 1) / BK;
  const int kb_begin = split * kb_per_split, kb_end = min(num_kb, kb_begin + kb_per_split);
  const int my_kb = max(0, kb_end - kb_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"((uint32_t)(TOK < 32 ? 32 : TOK))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < my_kb; ++i) {
        const int stage = i % STAGES;
        if (!mbar_wait(empty_bar(stage), ((i / STAGES) & 1) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t sw = base + stage * C::STAGE_BYTES, sx = sw + W_BYTES;
        mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
        tma_load_2d(sw, &map_w, full_bar(stage), (kb_begin + i) * BK, n0);
        tma_load_2d(sx, &map_x, full_bar(stage), (kb_begin + i) * BK, 0);
      }
      if (!ok) {
        atomicMax(status, ERR_SK_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BF, TOK, false, false);
      const uint32_t w_lo0 = desc_lo(base, true, 0), x_lo0 = desc_lo(base + W_BYTES, true, 0);
      bool ok = true;
      for (int i = 0; i < my_kb; ++i) {
        const int stage = i % STAGES;
        if (!mbar_wait(full_bar(stage), (i / STAGES) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t w_lo = w_lo0 + stage * (C::STAGE_BYTES >> 4), x_lo = x_lo0 + stage * (C::STAGE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) tc_mma_lo(tmem_base, w_lo + 2 * k, x_lo + 2 * k, idesc, (i | k) ? 1u : 0u);
        tc_commit(empty_bar(stage));
      }
      if (ok) tc_commit(done_bar);
      else {
        atomicMax(status, ERR_SK_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    // epilogue warps: lane = output feature, TMEM columns = tokens.  Park the fp32 tile as [token][feature] in the
    // (now idle) ring: the commit behind `done_bar` fires after every MMA - hence every TMA write - has retired.
    const int quarter = warp & 3;
    const int fl = quarter * 32 + lane;
    float* red = reinterpret_cast<float*>(aligned);
    const bool ok = __all_sync(0xffffffffu, mbar_wait(done_bar, 0, abort_flag));
    if (ok) tc_fence_after();
#pragma unroll
    for (int c = 0; c < TOK / 16; ++c) {
      uint32_t r[16];
      if (ok && my_kb > 0) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16)
            : "memory");
        tc_wait_ld();
      } else {
#pragma unroll
        for (int t = 0; t < 16; ++t) r[t] = 0u;
      }
#pragma unroll
      for (int t = 0; t < 16; ++t) red[(c * 16 + t) * BF + fl] = __uint_as_float(r[t]);
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR_SK_EPILOGUE);
      *abort_flag = 1;
    }
  }

  // ---- cluster-wide reduction through distributed shared memory: CTA `split` owns every cs-th group of 4 features
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  {
    const uint32_t red_addr = base;  // same offset in every CTA of the cluster
    const int vec_total = M * (BF / 4);
    for (int v = split * NUM_THREADS + threadIdx.x; v < vec_total; v += cs * NUM_THREADS) {
      const int t = v / (BF / 4), f4 = (v % (BF / 4)) * 4;
      // all peers' loads are issued before the first add: distributed-shared-memory latency is paid once per vector
      float4 p[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < cs) p[c] = ld_dsmem_f4(mapa(red_addr + (uint32_t)(t * BF + f4) * 4u, (uint32_t)c));
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < cs) acc.x += p[c].x, acc.y += p[c].y, acc.z += p[c].z, acc.w += p[c].w;
      const int f = n0 + f4;
      __nv_bfloat16* dst = Y + (long long)t * ldy + f;
      if (f + 4 <= N && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = pk;
      } else {
        const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
        for (int j = 0; j < 4 && f + j < N; ++j) dst[j] = __float2bfloat16_rn(a4[j]);
      }
    }
  }
  cluster_sync();  // nobody leaves while a peer may still read its shared memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(TOK < 32 ? 32 : TOK)) : "memory");
  }
}

template <int TOK>
int launch_sk(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, int M, int N, int K, long long ldy, int cs, int kb_per_split,
              int* status, cudaStream_t st) {
  auto kern = gemm_skinny_kernel<TOK>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SkCfg<TOK>::SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(((N + BF - 1) / BF) * cs, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SkCfg<TOK>::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  __nv_bfloat16* y = (__nv_bfloat16*)Y;
  return cudaLaunchKernelEx(&cfg, kern, mw, mx, y, M, N, K, ldy, kb_per_split, status) == cudaSuccess ? 0 : -5;
}

}  // namespace

// CTAs per feature tile (cluster size): enough CTAs to cover the machine, at least two K blocks each.
int gemm_skinny_splits(int N, int K, int tok) {
  const int tiles = (N + BF - 1) / BF, num_kb = (K + BK - 1) / BK;
  const int limit = tok <= 64 ? 300 : 148;  // two CTAs fit on an SM up to 64 tokens, one above: stay within one wave
  int cs = 1;
  while (cs < 8 && tiles * cs * 2 <= limit && num_kb / (cs * 2) >= 2) cs *= 2;
  return cs;
}

int gemm_skinny(const void* X, const void* W, void* Y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
                int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 256) return -6;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldx % 8) || (ldw % 8)) return -1;
  const int tok = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
  const int num_kb = (K + BK - 1) / BK;
  const int cs = gemm_skinny_splits(N, K, tok);
  const int kb_per_split = (num_kb + cs - 1) / cs;
  CUtensorMap mw, mx;
  if (!cache().get(&mw, W, K, N, ldw, BK, BF)) return -1000 - g_last_map_error;
  if (!cache().get(&mx, X, K, M, ldx, BK, tok)) return -2000 - g_last_map_error;
  switch (tok) {
    case 16: return launch_sk<16>(mw, mx, Y, M, N, K, ldy, cs, kb_per_split, status, st);
    case 32: return launch_sk<32>(mw, mx, Y, M, N, K, ldy, cs, kb_per_split, status, st);
    case 64: return launch_sk<64>(mw, mx, Y, M, N, K, ldy, cs, kb_per_split, status, st);
    case 128: return launch_sk<128>(mw, mx, Y, M, N, K, ldy, cs, kb_per_split, status, st);
    default: return launch_sk<256>(mw, mx, Y, M, N, K, ldy, cs, kb_per_split, status, st);
  }
}

}  // namespace ab
