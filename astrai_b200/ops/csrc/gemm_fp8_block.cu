// Block-scaled fp8 (E4M3) GEMM on tcgen05: one fp32 scale per 1 x 128 block of the activations and per 128 x 128 block
// of the weights,  D[m, n] = sum_kb sa[m, kb] * sb[n / 128, kb] * (A_q[m, kb-block] . B_q[n, kb-block]).
//
// The hardware's own block scaling (kind::mxf8f6f4) uses 32-element blocks with power-of-two scales; scales of
// granularity 128 in fp32 have to be applied to partial sums instead.  The 128-wide K block of the quantisation is
// exactly one pipeline stage (128 bytes = one 128-byte-swizzle atom per row, four K = 32 MMAs), so:
//   warp 0      : TMA producer, 6-stage ring of A [128 x 128 B] and B [128 x 128 B] tiles
//   warp 1      : MMA issuer - every K block goes into a FRESH accumulator: one of four 128-column TMEM buffers
//   warps 2..9  : promotion + epilogue - each thread owns one output row and 64 of the tile's 128 columns in registers;
//                 per K block it reads the partial sums of its row (tcgen05.ld), releases the TMEM buffer, and adds
//                 them times sa[row, kb] * sb[tile, kb]; at the end of the K loop it writes bf16.
// Four TMEM buffers let the tensor core run up to three K blocks ahead of the promotion warps; eight warps (two per
// TMEM lane quarter, splitting the columns) keep the promotion at about the pace of the MMAs.
// Layout of the scales: sa_t [K / 128, M] (block-major, so a warp's 32 rows read 128 contiguous bytes), sb [ceil(N / 128), K / 128].
// The reference's fp8 path is per-tensor only (csrc/kernels/fp8/mm.cu:49-54 rejects anything but one scale per operand).
// Every mbarrier wait is bounded; expiry records a code in `status`.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

using namespace tc;
using namespace tmah;

constexpr int BM = 128, BN = 128, BKB = 128, STAGES = 6, UMMA_K = 32, PBUF = 4;
constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 320;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
enum : int { ERR_FB_PRODUCER = 91, ERR_FB_MMA = 92, ERR_FB_EPILOGUE = 93 };

__host__ __device__ constexpr uint32_t idesc_e4m3(int M, int N) {  // kind::f8f6f4, fp32 accumulator, E4M3 x E4M3, K-major
  return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(DESC_HI), "r"(0u)
      : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      __nv_bfloat16* __restrict__ D, const float* __restrict__ sa_t, const float* __restrict__ sb,
                      const __nv_bfloat16* __restrict__ bias, int M, int N, int K, long long ldd, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + STAGES * STAGE_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto pfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto pempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + PBUF + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * PBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, num_tiles = tiles_m * tiles_n;
  const int num_kb = K / BKB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < PBUF; ++b) {
      mbar_init(pfull_bar(b), 1);
      mbar_init(pempty_bar(b), 8);
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
  auto coord = [&](int t, int& m0, int& n0) {  // row tiles vary fastest inside groups of 16: the B tile stays in L2
    constexpr int G = 16;
    const int per_group = G * tiles_n, g = t / per_group, r = t % per_group;
    const int rows = min(G, tiles_m - g * G);
    m0 = (g * G + r % rows) * BM;
    n0 = (r / rows) * BN;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0;
        coord(t, m0, n0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES, sbm = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &map_a, full_bar(stage), kb * BKB, m0);
          tma_load_2d(sbm, &map_b, full_bar(stage), kb * BKB, n0);
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_FB_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_e4m3(BM, BN);
      const uint32_t a_lo0 = desc_lo(base, true, 0), b_lo0 = desc_lo(base + A_BYTES, true, 0);
      int stage = 0, pb = 0;
      uint32_t phase = 0, pphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag) || !mbar_wait(pempty_bar(pb), pphase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
          const uint32_t d_tmem = tmem_base + pb * BN;
#pragma unroll
          for (int k = 0; k < BKB / UMMA_K; ++k) mma_f8(d_tmem, a_lo + 2 * k, b_lo + 2 * k, idesc, k ? 1u : 0u);
          tc_commit(empty_bar(stage));
          tc_commit(pfull_bar(pb));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
          if (++pb == PBUF) pb = 0, pphase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_FB_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;  // TMEM lane quarter, column half of the tile
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 64;
    int pb = 0;
    uint32_t pphase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m0, n0;
      coord(t, m0, n0);
      const int row = m0 + quarter * 32 + lane;
      const bool live = row < M;
      const float* sa_row = sa_t + (live ? row : 0);
      const float* sb_row = sb + (long long)(n0 / BN) * num_kb;
      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      float s_next = live ? __ldg(sa_row) * __ldg(sb_row) : 0.f;
      for (int kb = 0; kb < num_kb; ++kb) {
        const float s = s_next;
        if (kb + 1 < num_kb) s_next = live ? __ldg(sa_row + (long long)(kb + 1) * M) * __ldg(sb_row + kb + 1) : 0.f;
        if (!__all_sync(0xffffffffu, mbar_wait(pfull_bar(pb), pphase, abort_flag))) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t v0[32], v1[32];
        tc_ld32(t_lane + pb * BN, v0);
        tc_ld32(t_lane + pb * BN + 32, v1);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pempty_bar(pb));  // the partial sums are in registers: the buffer may be overwritten
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = fmaf(__uint_as_float(v0[i]), s, acc[i]);
          acc[32 + i] = fmaf(__uint_as_float(v1[i]), s, acc[32 + i]);
        }
        if (++pb == PBUF) pb = 0, pphase ^= 1u;
      }
      if (!ok) break;
      const int col0 = n0 + half * 64;
      if (live && col0 < N) {
        __nv_bfloat16* d = D + (long long)row * ldd + col0;
        const bool vec = (col0 + 64 <= N) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
        if (vec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 pk;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float lo = acc[8 * j + 2 * q], hi = acc[8 * j + 2 * q + 1];
              if (bias) lo += __bfloat162float(bias[col0 + 8 * j + 2 * q]), hi += __bfloat162float(bias[col0 + 8 * j + 2 * q + 1]);
              const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
              pw[q] = *reinterpret_cast<const uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(d)[j] = pk;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (col0 + j < N) d[j] = __float2bfloat16_rn(acc[j] + (bias ? __bfloat162float(bias[col0 + j]) : 0.f));
        }
      }
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR_FB_EPILOGUE);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// 1 x 128 blocks: 16 threads (8 elements each) per block; the scale goes to sa_t[kb, row].
__global__ void fp8_quantize_act_block_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ sa_t,
                                              int rows, int cols, long long ldx) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = cols / 8;
  const long long r = gid / per_row;
  const int c = (int)(gid % per_row) * 8;
  float f[8];
  float mx = 0.f;
  const bool in = r < rows;
  if (in) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x, f[2 * i + 1] = t.y;
      mx = fmaxf(mx, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));  // 16 lanes = one 128-wide block
  if (!in) return;
  const float scale = mx > 0.f ? mx / 448.f : 1.f, inv = 1.f / scale;
  uint8_t b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = (uint8_t)__nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint2*>(q + r * cols + c) = *reinterpret_cast<const uint2*>(b);
  if ((c & 127) == 0) sa_t[(long long)(c >> 7) * rows + r] = scale;
}

// 128 x 128 blocks: one CTA of 256 threads per block.
__global__ void __launch_bounds__(256)
fp8_quantize_weight_block_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, float* __restrict__ sb, int rows,
                                 int cols, long long ldw) {
  __shared__ float s_max[8];
  __shared__ float s_scale;
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 128;
  const int tr = threadIdx.x >> 4, tc8 = (threadIdx.x & 15) * 8;  // 16 rows x 16 chunks per pass, 8 passes
  float mx = 0.f;
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
    const int r = r0 + tr + pass * 16;
    if (r < rows) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + (long long)r * ldw + c0 + tc8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        mx = fmaxf(mx, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, s_max[i]);
    s_scale = m > 0.f ? m / 448.f : 1.f;
    sb[(long long)blockIdx.y * gridDim.x + blockIdx.x] = s_scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
    const int r = r0 + tr + pass * 16;
    if (r < rows) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + (long long)r * ldw + c0 + tc8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      uint8_t b[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        b[2 * i] = (uint8_t)__nv_cvt_float_to_fp8(t.x * inv, __NV_SATFINITE, __NV_E4M3);
        b[2 * i + 1] = (uint8_t)__nv_cvt_float_to_fp8(t.y * inv, __NV_SATFINITE, __NV_E4M3);
      }
      *reinterpret_cast<uint2*>(q + (long long)r * cols + c0 + tc8) = *reinterpret_cast<const uint2*>(b);
    }
  }
}

bool map_u8(CUtensorMap* out, const void* ptr, long long inner, long long outer, int box_inner, int box_outer) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)inner};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_map_error = (int)res;
  return res == CUDA_SUCCESS;
}

}  // namespace

int fp8_quantize_act_block(const void* x, void* q, float* sa_t, int rows, int cols, long long ldx, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 128 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return -1;
  const long long threads = (long long)rows * (cols / 8);
  fp8_quantize_act_block_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, sa_t, rows, cols, ldx);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int fp8_quantize_weight_block(const void* w, void* q, float* sb, int rows, int cols, long long ldw, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 128 || ldw % 8 || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return -1;
  const dim3 grid(cols / 128, (rows + 127) / 128);
  fp8_quantize_weight_block_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, (uint8_t*)q, sb, rows, cols, ldw);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int gemm_fp8_block(const void* A, const void* B, void* D, const float* sa_t, const float* sb, const void* bias, int M, int N, int K,
                   long long ldd, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (K % 128)) return -1;
  CUtensorMap ma, mb;
  if (!map_u8(&ma, A, K, M, BKB, BM)) return -1000 - g_last_map_error;
  if (!map_u8(&mb, B, K, N, BKB, BN)) return -2000 - g_last_map_error;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  gemm_fp8_block_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, (__nv_bfloat16*)D, sa_t, sb, (const __nv_bfloat16*)bias, M, N, K, ldd,
                                                               status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
