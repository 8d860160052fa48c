// Mixture-of-experts routing and token movement (sm_100a), all on the device - no host synchronisation per layer.
//
//   moe_router      : softmax over E experts (fp32), top-k (k <= 8) by repeated warp arg-max, optional renormalisation
//                     of the k weights, per-expert token counts and probability sums (auxiliary load-balance loss).
//                     One warp per token, E <= 256.
//   moe_plan        : counts -> segment offsets padded to 128 rows (so a 128-row GEMM tile never straddles two
//                     experts and the K blocks of the ragged weight-gradient never mix experts), the tile -> expert
//                     map read by the grouped GEMM, and the total padded row count.
//   moe_permute     : copies every (token, choice) row into its expert's segment (slot = offset + atomic cursor),
//                     records the slot, and zero-fills the padding rows.
//   moe_combine     : out[t] = sum_k w[t,k] * y[slot[t,k]]  (a gather: deterministic, no atomics); its backward
//                     pieces (scatter of w * dout into slots, <dout, y> per choice) are moe_combine_bwd.
//   moe_gather_sum  : dx[t] = sum_k dxs[slot[t,k]]  (backward of the permutation).
// These replace softmax / topk / sort / bincount / index_add_ plus a Python loop over experts with a `.tolist()` host
// sync per layer in the reference (astrai/model/components/mlp.py:124-166).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "launchers.h"

namespace ab {
namespace {

constexpr int MAX_E = 256, MAX_K = 8;

template <typename T>
__global__ void __launch_bounds__(256)
moe_router_kernel(const T* __restrict__ logits, T* __restrict__ probs, long long* __restrict__ idx, T* __restrict__ weights,
                  int* __restrict__ counts, float* __restrict__ probsum, long long tokens, int E, int K, int renorm) {
  __shared__ int s_cnt[MAX_E];
  __shared__ float s_sum[MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0, s_sum[e] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  constexpr int PER = MAX_E / 32;
  for (long long t = (long long)blockIdx.x * warps + (threadIdx.x >> 5); t < tokens; t += (long long)gridDim.x * warps) {
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      v[i] = e < E ? to_f(logits[t * E + e]) : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      // the reference rounds the probabilities to the activation dtype before top-k (mlp.py:124-126)
      v[i] = e < E ? to_f(from_f<T>(v[i] * inv)) : -1.f;
      if (e < E) {
        probs[t * E + e] = from_f<T>(v[i]);
        atomicAdd(&s_sum[e], v[i]);
      }
    }
    float wk[MAX_K];
    int ek[MAX_K];
    float wsum = 0.f;
    for (int k = 0; k < K; ++k) {
      float best = -2.f;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        if (v[i] > best || (v[i] == best && e < be)) best = v[i], be = e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ob > best || (ob == best && oe < be)) best = ob, be = oe;
      }
      wk[k] = best, ek[k] = be, wsum += best;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i * 32 + lane == be) v[i] = -1.f;  // taken
    }
    if (lane == 0) {
      const float sc = renorm ? 1.f / wsum : 1.f;
      for (int k = 0; k < K; ++k) {
        idx[t * K + k] = ek[k];
        weights[t * K + k] = from_f<T>(to_f(from_f<T>(wk[k])) * sc);
        atomicAdd(&s_cnt[ek[k]], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_cnt[e]) atomicAdd(&counts[e], s_cnt[e]);
    if (s_sum[e] != 0.f) atomicAdd(&probsum[e], s_sum[e]);
  }
}

// One CTA.  offsets[E+1] (padded to 128), tile_expert[max_tiles] (-1 past the end), cursors[E] = 0, total[0] = padded rows.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ tile_expert,
                                int* __restrict__ cursors, int* __restrict__ total, int E, int max_tiles) {
  __shared__ int s_off[MAX_E + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = acc;
    total[0] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E) cursors[e] = 0;
  }
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * 128;
    int lo = 0, hi = E;  // last e with s_off[e] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_off[mid] <= row) lo = mid; else hi = mid;
    }
    tile_expert[t] = (row < s_off[E] && row < s_off[lo + 1]) ? lo : -1;
  }
}

template <typename T>
__global__ void moe_permute_kernel(const T* __restrict__ x, const long long* __restrict__ idx, const int* __restrict__ offsets,
                                   int* __restrict__ cursors, T* __restrict__ sorted, int* __restrict__ slot_of, long long tokens,
                                   int K, int D) {
  // one warp per (token, choice)
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= tokens * K) return;
  const long long t = w / K;
  const int e = (int)idx[w];
  int slot = 0;
  if (lane == 0) {
    slot = offsets[e] + atomicAdd(&cursors[e], 1);
    slot_of[w] = slot;
  }
  slot = __shfl_sync(0xffffffffu, slot, 0);
  const uint4* src = reinterpret_cast<const uint4*>(x + t * D);
  uint4* dst = reinterpret_cast<uint4*>(sorted + (long long)slot * D);
  constexpr int PER16 = 16 / sizeof(T);
  for (int i = lane; i < D / PER16; i += 32) dst[i] = src[i];
}

template <typename T>
__global__ void moe_zero_pad_kernel(T* __restrict__ sorted, const int* __restrict__ counts, const int* __restrict__ offsets, int E,
                                    int D) {
  // block (e, chunk): zero the rows [offsets[e] + counts[e], offsets[e+1])
  const int e = blockIdx.x;
  const int begin = offsets[e] + counts[e], end = offsets[e + 1];
  constexpr int PER16 = 16 / sizeof(T);
  const long long vecs = (long long)(end - begin) * (D / PER16);
  uint4* base = reinterpret_cast<uint4*>(sorted + (long long)begin * D);
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.y * blockDim.x)
    base[i] = make_uint4(0, 0, 0, 0);
}

// out[t] = sum_k w[t,k] * y[slot[t,k]]   (one warp per token, eight elements per lane trip)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ slot_of, const T* __restrict__ weights,
                                   T* __restrict__ out, long long tokens, int K, int D, int use_w) {
  const long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  for (int c = lane * 8; c < D; c += 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < K; ++k) {
      const float w = use_w ? to_f(weights[t * K + k]) : 1.f;
      Vec8<T> v;
      v.load(y + (long long)slot_of[t * K + k] * D + c);
      float f[8];
      v.unpack(f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * f[j];
    }
    Vec8<T> o;
    o.pack(acc);
    o.store(out + t * D + c);
  }
}

// dy[slot[t,k]] = w[t,k] * dout[t];  dw[t,k] = <dout[t], y[slot[t,k]]>   (one warp per (token, choice))
template <typename T>
__global__ void moe_combine_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ y, const int* __restrict__ slot_of,
                                       const T* __restrict__ weights, T* __restrict__ dy, float* __restrict__ dw,
                                       long long tokens, int K, int D) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= tokens * K) return;
  const long long t = w / K;
  const int slot = slot_of[w];
  const float wt = to_f(weights[w]);
  float dot = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    Vec8<T> g, v;
    g.load(dout + t * D + c);
    v.load(y + (long long)slot * D + c);
    float gf[8], vf[8], of[8];
    g.unpack(gf);
    v.unpack(vf);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += gf[j] * vf[j], of[j] = wt * gf[j];
    Vec8<T> o;
    o.pack(of);
    o.store(dy + (long long)slot * D + c);
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[w] = dot;
}

}  // namespace

#define AB_DISPATCH_T(is_bf16, ...)           \
  if (is_bf16) {                              \
    using T = __nv_bfloat16;                  \
    __VA_ARGS__;                              \
  } else {                                    \
    using T = float;                          \
    __VA_ARGS__;                              \
  }

int moe_router(const void* logits, void* probs, long long* idx, void* weights, int* counts, float* probsum, long long tokens,
               int E, int K, bool renorm, bool is_bf16, cudaStream_t st) {
  if (E < 1 || E > MAX_E || K < 1 || K > MAX_K || K > E) return -1;
  if (tokens == 0) return 0;
  long long blocks = (tokens + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  AB_DISPATCH_T(is_bf16, (moe_router_kernel<T><<<(int)blocks, 256, 0, st>>>((const T*)logits, (T*)probs, idx, (T*)weights, counts, probsum,
                                                                          tokens, E, K, renorm ? 1 : 0)));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_plan(const int* counts, int* offsets, int* tile_expert, int* cursors, int* total, int E, int max_tiles, cudaStream_t st) {
  if (E < 1 || E > MAX_E) return -1;
  moe_plan_kernel<<<1, 256, 0, st>>>(counts, offsets, tile_expert, cursors, total, E, max_tiles);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_permute(const void* x, const long long* idx, const int* counts, const int* offsets, int* cursors, void* sorted, int* slot_of,
                long long tokens, int K, int D, int E, bool is_bf16, cudaStream_t st) {
  if (D % 8) return -1;
  if (tokens == 0) return 0;
  const long long warps = tokens * K;
  AB_DISPATCH_T(is_bf16, (moe_zero_pad_kernel<T><<<dim3(E, 4), 256, 0, st>>>((T*)sorted, counts, offsets, E, D)));
  AB_DISPATCH_T(is_bf16, (moe_permute_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>((const T*)x, idx, offsets, cursors, (T*)sorted,
                                                                                                   slot_of, tokens, K, D)));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_combine(const void* y, const int* slot_of, const void* weights, void* out, long long tokens, int K, int D, bool is_bf16,
                cudaStream_t st) {
  if (D % 8) return -1;
  if (tokens == 0) return 0;
  AB_DISPATCH_T(is_bf16, (moe_combine_kernel<T><<<(unsigned)((tokens * 32 + 255) / 256), 256, 0, st>>>((const T*)y, slot_of, (const T*)weights, (T*)out,
                                                                                                    tokens, K, D, weights != nullptr)));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int moe_combine_bwd(const void* dout, const void* y, const int* slot_of, const void* weights, void* dy, float* dw, long long tokens,
                    int K, int D, bool is_bf16, cudaStream_t st) {
  if (D % 8) return -1;
  if (tokens == 0) return 0;
  const long long warps = tokens * K;
  AB_DISPATCH_T(is_bf16, (moe_combine_bwd_kernel<T><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>((const T*)dout, (const T*)y, slot_of,
                                                                                                       (const T*)weights, (T*)dy, dw, tokens, K, D)));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
