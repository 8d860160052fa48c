// Fused FSDP kernels over NVLink peer memory (one process per GPU, symmetric buffers mapped into every rank).
//
//   fsdp_reduce_scatter : gradient reduce-scatter + squared-norm partial in ONE kernel.  The owner of a shard pulls
//       that shard of the fp32 gradient buffer from every rank (16-byte coherent peer loads, fixed rank order so the
//       sum is reproducible; or one multimem.ld_reduce per 16 bytes, summed inside NVSwitch), writes the reduced
//       shard locally and adds sum(g^2) to the clip-norm accumulator.  Readiness of the peers' gradients is
//       signalled through flags with bounded waits - no NCCL call, no separate norm pass.
//   fsdp_adamw_allgather : cast/scale (clip coefficient x 1/world from a device scalar) + AdamW on the owned shard
//       (fp32 moments and master weights) + parameter all-gather in ONE kernel: the updated bf16 values are stored
//       straight into every rank's parameter buffer (peer stores, or one multimem.st), followed by a per-unit
//       "written" flag that the next forward pass waits on.
//   comm_wait_flags : the consumer side of such a flag (one tiny CTA on the compute stream).
// These replace FSDP2's all-gather / reduce-scatter + clip_grad_norm_ + AdamW sequence of the reference
// (astrai/parallel/executor.py:343-399, astrai/optim/muon_adamw.py:69-74).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"
#include "launchers.h"

namespace ab {
namespace {

using namespace comm;

constexpr int THREADS = 256;

// Flag word written by rank `src` on the rank that owns `base`: [kind][src][unit].
__device__ __forceinline__ int* flag_slot(void* base, int kind, int src, int unit, int max_units) {
  return reinterpret_cast<int*>(base) + ((long long)kind * MAX_RANKS + src) * max_units + unit;
}

template <bool MC>
__global__ void __launch_bounds__(THREADS)
fsdp_rs_kernel(CommPeers grads, const float* __restrict__ mc_grads, CommPeers flags, int world, int rank,
               long long shard_off, long long n, float* __restrict__ out, float* __restrict__ sumsq, int unit,
               int max_units, int epoch, unsigned long long timeout_ns, int* __restrict__ status) {
  __shared__ int s_ok;
  __shared__ float s_red[THREADS / 32];
  if (threadIdx.x == 0) s_ok = 1;
  // This rank's gradients of the unit are complete (stream order): tell every rank, then wait for theirs.
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flag_slot(flags.ptr[threadIdx.x], 0, rank, unit, max_units), epoch);
  }
  __syncthreads();
  if (threadIdx.x < world && threadIdx.x != rank) {
    if (!wait_flag(flag_slot(flags.ptr[rank], 0, threadIdx.x, unit, max_units), epoch, timeout_ns)) {
      atomicMax(status, ERR_WAIT_PEER_READY);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) return;

  float acc = 0.f;
  const long long nvec = n >> 2;
  constexpr int U = 4;  // independent 16-byte loads in flight per rank and thread (NVLink latency is ~2 us)
  const long long stride = (long long)gridDim.x * THREADS;
  for (long long i0 = (long long)blockIdx.x * THREADS + threadIdx.x; i0 < nvec; i0 += stride * U) {
    float4 s[U];
    if (MC) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < nvec) s[u] = mc_ld_reduce_f4(mc_grads + shard_off + 4 * (i0 + u * stride));
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < MAX_RANKS; ++p) {
        if (p < world) {
          float4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * stride < nvec)
              v[u] = ld_sys_f4(reinterpret_cast<const float*>(grads.ptr[p]) + shard_off + 4 * (i0 + u * stride));
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * stride < nvec) s[u].x += v[u].x, s[u].y += v[u].y, s[u].z += v[u].z, s[u].w += v[u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i0 + u * stride < nvec) {
        reinterpret_cast<float4*>(out)[i0 + u * stride] = s[u];
        acc += s[u].x * s[u].x + s[u].y * s[u].y + s[u].z * s[u].z + s[u].w * s[u].w;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && sumsq != nullptr) {
    float t = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) t += s_red[w];
    atomicAdd(sumsq, t);
  }
}

template <bool MC>
__global__ void __launch_bounds__(THREADS)
fsdp_adamw_ag_kernel(CommPeers params, __nv_bfloat16* __restrict__ mc_params, CommPeers flags, int world, int rank,
                     long long shard_off, long long n, float* __restrict__ master, const float* __restrict__ g,
                     float* __restrict__ m, float* __restrict__ v, float lr, float b1, float b2, float eps, float wd,
                     float bc1, float bc2_sqrt, const float* __restrict__ gscale, int unit, int max_units, int epoch,
                     int* __restrict__ block_counter) {
  const float gs = gscale ? *gscale : 1.f;
  const long long nvec = n >> 3;  // eight elements = one 16-byte bf16 store per rank
  __nv_bfloat16* own = reinterpret_cast<__nv_bfloat16*>(params.ptr[rank]) + shard_off;
  for (long long i = (long long)blockIdx.x * THREADS + threadIdx.x; i < nvec; i += (long long)gridDim.x * THREADS) {
    float gr[8], mm[8], vv[8], w[8];
    *reinterpret_cast<float4*>(gr) = reinterpret_cast<const float4*>(g)[2 * i];
    *reinterpret_cast<float4*>(gr + 4) = reinterpret_cast<const float4*>(g)[2 * i + 1];
    *reinterpret_cast<float4*>(mm) = reinterpret_cast<const float4*>(m)[2 * i];
    *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<const float4*>(m)[2 * i + 1];
    *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(v)[2 * i];
    *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(v)[2 * i + 1];
    if (master) {
      *reinterpret_cast<float4*>(w) = reinterpret_cast<const float4*>(master)[2 * i];
      *reinterpret_cast<float4*>(w + 4) = reinterpret_cast<const float4*>(master)[2 * i + 1];
    } else {
      const uint4 raw = reinterpret_cast<const uint4*>(own)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(h[j]);
        w[2 * j] = t.x, w[2 * j + 1] = t.y;
      }
    }
    uint4 packed;
    __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float grad = gr[j] * gs;
      mm[j] = b1 * mm[j] + (1.f - b1) * grad;
      vv[j] = b2 * vv[j] + (1.f - b2) * grad * grad;
      w[j] *= (1.f - lr * wd);
      w[j] -= (lr / bc1) * mm[j] / (sqrtf(vv[j]) / bc2_sqrt + eps);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) ph[j] = __floats2bfloat162_rn(w[2 * j], w[2 * j + 1]);
    reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mm);
    reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
    reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
    reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
    if (master) {
      reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(w);
      reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(w + 4);
    }
    if (MC) {
      mc_st_u4(mc_params + shard_off + 8 * i, packed);
    } else {
#pragma unroll
      for (int p = 0; p < MAX_RANKS; ++p)
        if (p < world) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[p]) + shard_off)[i] = packed;
    }
  }
  // Last CTA out publishes "this rank's shard of the unit is written everywhere".
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(block_counter, 1);
    s_last = (done == (int)gridDim.x - 1);
    if (s_last) *block_counter = 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flag_slot(flags.ptr[threadIdx.x], 1, rank, unit, max_units), epoch);
  }
}

__global__ void comm_wait_kernel(const int* __restrict__ local_flags, int kind, int world, int skip_rank, int unit,
                                 int max_units, int epoch, unsigned long long timeout_ns, int* __restrict__ status) {
  if (threadIdx.x < world && threadIdx.x != skip_rank) {
    const int* f = local_flags + ((long long)kind * MAX_RANKS + threadIdx.x) * max_units + unit;
    if (!wait_flag(f, epoch, timeout_ns)) atomicMax(status, ERR_WAIT_FLAG);
  }
}

int grid_for(long long vecs, int max_ctas) {
  long long g = (vecs + THREADS - 1) / THREADS;
  if (g > max_ctas) g = max_ctas;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace

int fsdp_reduce_scatter(const CommPeers& grads, const float* mc_grads, const CommPeers& flags, int world, int rank,
                        long long shard_off, long long n, float* out, float* sumsq, int unit, int max_units, int epoch,
                        unsigned long long timeout_ns, int* status, int max_ctas, cudaStream_t st) {
  if (world < 1 || world > comm::MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (n % 4 || shard_off % 4 || unit < 0 || unit >= max_units) return -2;
  const int grid = grid_for(n >> 2, max_ctas);
  if (mc_grads)
    fsdp_rs_kernel<true><<<grid, THREADS, 0, st>>>(grads, mc_grads, flags, world, rank, shard_off, n, out, sumsq, unit,
                                                   max_units, epoch, timeout_ns, status);
  else
    fsdp_rs_kernel<false><<<grid, THREADS, 0, st>>>(grads, nullptr, flags, world, rank, shard_off, n, out, sumsq, unit,
                                                    max_units, epoch, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int fsdp_adamw_allgather(const CommPeers& params, void* mc_params, const CommPeers& flags, int world, int rank,
                         long long shard_off, long long n, float* master, const float* g, float* m, float* v, float lr,
                         float b1, float b2, float eps, float wd, int step, const float* gscale, int unit,
                         int max_units, int epoch, int* block_counter, int max_ctas, cudaStream_t st) {
  if (world < 1 || world > comm::MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (n % 8 || shard_off % 8 || unit < 0 || unit >= max_units) return -2;
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2_sqrt = sqrtf(1.f - powf(b2, (float)step));
  const int grid = grid_for(n >> 3, max_ctas);
  if (mc_params)
    fsdp_adamw_ag_kernel<true><<<grid, THREADS, 0, st>>>(params, (__nv_bfloat16*)mc_params, flags, world, rank,
                                                         shard_off, n, master, g, m, v, lr, b1, b2, eps, wd, bc1,
                                                         bc2_sqrt, gscale, unit, max_units, epoch, block_counter);
  else
    fsdp_adamw_ag_kernel<false><<<grid, THREADS, 0, st>>>(params, nullptr, flags, world, rank, shard_off, n, master, g,
                                                          m, v, lr, b1, b2, eps, wd, bc1, bc2_sqrt, gscale, unit,
                                                          max_units, epoch, block_counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int comm_wait_flags(const int* local_flags, int kind, int world, int skip_rank, int unit, int max_units, int epoch,
                    unsigned long long timeout_ns, int* status, cudaStream_t st) {
  if (world < 1 || world > comm::MAX_RANKS || unit < 0 || unit >= max_units) return -1;
  comm_wait_kernel<<<1, 32, 0, st>>>(local_flags, kind, world, skip_rank, unit, max_units, epoch, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
