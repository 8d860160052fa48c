// FP8 (E4M3 / E5M2) GEMM and quantisation for sm_100a.
//
//   fp8_quantize : bf16 -> fp8 with a per-tensor scale read from the device (q = x / scale, saturating), the raw
//                  amax of the input recorded with one atomicMax per CTA, and - optionally - the TRANSPOSED fp8 tensor
//                  written in the same pass through a shared-memory tile, so that dgrad / wgrad get K-major
//                  operands without a separate transpose + re-quantise (the reference materialises
//                  `.transpose().contiguous()` copies and quantises them again, csrc/kernels/fp8/mm.cu:294-313).
//   gemm_fp8     : D[M,N] = (A[M,K] . B[N,K]^T) * scale_a * scale_b (+ bias), fp8 operands (any mix of E4M3 / E5M2),
//                  fp32 accumulation in TMEM, bf16 output.  Same persistent warp-specialised structure as the bf16
//                  kernel (TMA 4-stage ring of 128-byte-swizzled tiles, one MMA-issuing lane, double-buffered
//                  accumulator, four epilogue warps); tcgen05.mma kind::f8f6f4 consumes 32 K-elements per instruction.
//   gemm_int8      the same kernel instantiated for tcgen05.mma kind::i8: signed 8-bit operands, exact int32 accumulation
//                  in TMEM, epilogue D = acc * row_scale[m] * col_scale[n] (+ bias) - per-token activation scales and
//                  per-channel weight scales, both produced by int8_quantize_rows (symmetric, amax / 127 per row).
//                  The reference has no int8 path.
// These take the place of the reference's mma.sync m16n8k32 kernels (csrc/kernels/fp8/gemm.cuh:128-619).
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

// ------------------------------------------------------------------------------------------------ quantise
template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// One CTA handles a 64 x 64 tile: row-major output directly, transposed output through shared memory.
template <bool E5M2, bool WITH_T>
__global__ void __launch_bounds__(256)
fp8_quantize_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ qt,
                    const float* __restrict__ scale, float* __restrict__ amax, int rows, int cols, long long ldx) {
  __shared__ uint8_t tile[64][64 + 4];
  __shared__ float s_max[8];
  const float inv = 1.f / fmaxf(*scale, 1e-30f);
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tr = threadIdx.x >> 3, tc8 = (threadIdx.x & 7) * 8;  // 32 rows x 8 chunks of 8 columns per pass
  float mx = 0.f;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int r = r0 + tr + pass * 32, c = c0 + tc8;
    if (r < rows && c < cols) {
      float f[8];
      if (c + 8 <= cols && ((reinterpret_cast<uintptr_t>(x + (long long)r * ldx + c) & 15) == 0)) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + (long long)r * ldx + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t = __bfloat1622float2(h[i]);
          f[2 * i] = t.x, f[2 * i + 1] = t.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (c + i < cols) ? __bfloat162float(x[(long long)r * ldx + c + i]) : 0.f;
      }
      uint8_t b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        mx = fmaxf(mx, fabsf(f[i]));
        b[i] = to_fp8<E5M2>(f[i] * inv);
        if (WITH_T) tile[tr + pass * 32][tc8 + i] = b[i];
      }
      if (c + 8 <= cols && (cols % 8 == 0)) {
        *reinterpret_cast<uint2*>(q + (long long)r * cols + c) = *reinterpret_cast<const uint2*>(b);
      } else {
        for (int i = 0; i < 8 && c + i < cols; ++i) q[(long long)r * cols + c + i] = b[i];
      }
    } else if (WITH_T) {
#pragma unroll
      for (int i = 0; i < 8; ++i) tile[tr + pass * 32][tc8 + i] = 0;
    }
  }
  if (WITH_T) {
    __syncthreads();
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int tcol = tr + pass * 32;  // column of the input tile = row of the transposed output
      const int c = c0 + tcol, r = r0 + tc8;
      if (c < cols && r < rows) {
        uint8_t b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = tile[tc8 + i][tcol];
        if (r + 8 <= rows && (rows % 8 == 0)) {
          *reinterpret_cast<uint2*>(qt + (long long)c * rows + r) = *reinterpret_cast<const uint2*>(b);
        } else {
          for (int i = 0; i < 8 && r + i < rows; ++i) qt[(long long)c * rows + r + i] = b[i];
        }
      }
    }
  }
  if (amax != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = 0.f;
      for (int w = 0; w < 8; ++w) m = fmaxf(m, s_max[w]);
      atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));  // non-negative floats order like ints
    }
  }
}

// ------------------------------------------------------------------------------------------------ GEMM
constexpr int BM = 128, BN = 256, BKB = 128 /* K bytes = K elements per stage */, STAGES = 4, UMMA_K = 32;
constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
enum : int { ERR_F8_PRODUCER = 61, ERR_F8_MMA = 62, ERR_F8_EPILOGUE = 63 };

// kind::f8f6f4 instruction descriptor: fp32 accumulator, operand formats 0 = E4M3, 1 = E5M2, both K-major.
__host__ __device__ constexpr uint32_t idesc_fp8(int M, int N, int a_fmt, int b_fmt) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// kind::i8 instruction descriptor: int32 accumulator (D format 2), signed 8-bit operands (format 1), both K-major.
__host__ __device__ constexpr uint32_t idesc_i8(int M, int N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(DESC_HI), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(DESC_HI), "r"(0u)
      : "memory");
}

// I8 = false: fp8 operands, scale_a / scale_b point at one fp32 scalar each.
// I8 = true : int8 operands, scale_a is fp32 [M] (per row of A), scale_b fp32 [N] (per row of B = output column).
template <bool I8>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                __nv_bfloat16* __restrict__ D, const float* __restrict__ scale_a, const float* __restrict__ scale_b,
                const __nv_bfloat16* __restrict__ bias, int M, int N, int K, long long ldd, uint32_t idesc,
                int* __restrict__ status) {
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
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BKB - 1) / BKB;

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
  auto coord = [&](int t, int& m0, int& n0) {  // column tiles vary fastest inside groups of 16 row tiles
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
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &map_a, full_bar(stage), kb * BKB, m0);
          tma_load_2d(sb, &map_b, full_bar(stage), kb * BKB, n0);
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
      if (!ok) {
        atomicMax(status, ERR_F8_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t a_lo0 = desc_lo(base, true, 0), b_lo0 = desc_lo(base + A_BYTES, true, 0);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
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
          for (int k = 0; k < BKB / UMMA_K; ++k) {
            if (I8) tc_mma_i8(d_tmem, a_lo + 2 * k, b_lo + 2 * k, idesc, (kb | k) ? 1u : 0u);
            else tc_mma_f8(d_tmem, a_lo + 2 * k, b_lo + 2 * k, idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
      if (!ok) {
        atomicMax(status, ERR_F8_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const float sc_all = I8 ? 1.f : (*scale_a) * (*scale_b);
    auto val = [&](uint32_t bits, float sc, int col) {  // accumulator bits -> scaled fp32
      const float acc = I8 ? (float)(int)bits : __uint_as_float(bits);
      return acc * (I8 ? sc * scale_b[col] : sc);
    };
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const int buf = it & 1;
      int m0, n0;
      coord(t, m0, n0);
      if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const float sc = I8 ? (row < M ? scale_a[row] : 0.f) : sc_all;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld32(taddr0 + c * 32, r);
        tc_wait_ld();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          __nv_bfloat16* d = D + (long long)row * ldd + col;
          const bool vec = (col + 32 <= N) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
          if (vec) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float lo = val(r[8 * j + 2 * q], sc, col + 8 * j + 2 * q), hi = val(r[8 * j + 2 * q + 1], sc, col + 8 * j + 2 * q + 1);
                if (bias) lo += __bfloat162float(bias[col + 8 * j + 2 * q]), hi += __bfloat162float(bias[col + 8 * j + 2 * q + 1]);
                const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                pw[q] = *reinterpret_cast<const uint32_t*>(&h);
              }
              reinterpret_cast<uint4*>(d)[j] = pk;
            }
          } else {
            for (int j = 0; j < 32 && col + j < N; ++j) {
              float f = val(r[j], sc, col + j);
              if (bias) f += __bfloat162float(bias[col + j]);
              d[j] = __float2bfloat16_rn(f);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR_F8_EPILOGUE);
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

// 2-D uint8 tensor map with 128-byte swizzle (rows of `inner` bytes).
bool make_map_u8(CUtensorMap* out, const void* ptr, long long inner, long long outer, long long ld, int box_inner, int box_outer) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_map_error = (int)res;
  return res == CUDA_SUCCESS;
}

}  // namespace

int fp8_quantize(const void* x, void* q, void* qt, const float* scale, float* amax, int rows, int cols, long long ldx,
                 bool e5m2, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  const dim3 grid((cols + 63) / 64, (rows + 63) / 64);
#define AB_Q(E, T) \
  fp8_quantize_kernel<E, T><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)qt, scale, amax, rows, cols, ldx)
  if (e5m2) {
    if (qt) AB_Q(true, true); else AB_Q(true, false);
  } else {
    if (qt) AB_Q(false, true); else AB_Q(false, false);
  }
#undef AB_Q
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

namespace {

// One warp per row: amax over the row, scale = amax / 127 (1 for an all-zero row), q = round(x / scale) in [-127, 127].
__global__ void int8_quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale,
                                          int rows, int cols, long long ldx) {
  const int row = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (long long)row * ldx;
  float amax = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p[i]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / sc;
  if (lane == 0) scale[row] = sc;
  int8_t* qr = q + (long long)row * cols;
  for (int c = lane * 8; c < cols; c += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    int8_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p[i]);
      o[2 * i] = (int8_t)max(-127, min(127, __float2int_rn(f.x * inv)));
      o[2 * i + 1] = (int8_t)max(-127, min(127, __float2int_rn(f.y * inv)));
    }
    *reinterpret_cast<uint2*>(qr + c) = *reinterpret_cast<const uint2*>(o);
  }
}

template <bool I8>
int launch_q8(const void* A, const void* B, void* D, const float* scale_a, const float* scale_b, const void* bias, int M, int N,
              int K, long long ldd, uint32_t idesc, int* status, cudaStream_t st) {
  CUtensorMap ma, mb;
  if (!make_map_u8(&ma, A, K, M, K, BKB, BM)) return -1000 - g_last_map_error;
  if (!make_map_u8(&mb, B, K, N, K, BKB, BN)) return -2000 - g_last_map_error;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel<I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  gemm_fp8_kernel<I8><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, (__nv_bfloat16*)D, scale_a, scale_b, (const __nv_bfloat16*)bias,
                                                             M, N, K, ldd, idesc, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int int8_quantize_rows(const void* x, void* q, float* scale, int rows, int cols, long long ldx, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7)) return -1;
  const long long threads = (long long)rows * 32;
  int8_quantize_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, (int8_t*)q, scale, rows, cols, ldx);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int gemm_int8(const void* A, const void* B, void* D, const float* row_scale, const float* col_scale, const void* bias, int M,
              int N, int K, long long ldd, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (K % 16)) return -1;
  return launch_q8<true>(A, B, D, row_scale, col_scale, bias, M, N, K, ldd, idesc_i8(BM, BN), status, st);
}

int gemm_fp8(const void* A, const void* B, void* D, const float* scale_a, const float* scale_b, const void* bias, int M,
             int N, int K, long long ldd, bool a_e5m2, bool b_e5m2, int* status, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (K % 16)) return -1;
  return launch_q8<false>(A, B, D, scale_a, scale_b, bias, M, N, K, ldd, idesc_fp8(BM, BN, a_e5m2 ? 1 : 0, b_e5m2 ? 1 : 0), status, st);
}

}  // namespace ab
