// Token sampling on the device: temperature -> top-k -> top-p -> frequency penalty -> draw, one CTA per batch row.
//
// Semantics follow the reference's sampling pipeline (astrai/inference/runtime/sample.py:91-138, 178-232, 299-324):
//   * all temperatures exactly 0 (`all_greedy`): argmax of the raw logits, log-prob from the raw log-softmax;
//   * otherwise x = logit / max(temperature, 1e-8);
//   * top-k (k <= 0 or k >= V disables): values strictly below the k-th largest value are removed;
//   * top-p (p >= 1 disables): with tokens sorted by descending value, a token is removed when the probability mass
//     BEFORE it already exceeds p (the first crossing token stays; equal values at the crossing all stay);
//   * frequency penalty: x[token] -= penalty per occurrence of the token in the row's history (removed tokens stay removed);
//   * draw from softmax(x); the returned log-prob is log_softmax(x)[token] of that final distribution.
// Where the reference sorts the whole vocabulary (torch.topk / torch.sort / cumsum / scatter / multinomial, five
// kernels over [B, V] and as many temporaries), this kernel never sorts: the k-th largest value and the top-p crossing
// value are found by 4-pass radix selection on the order-preserving bit pattern of the floats (counts for top-k,
// probability mass for top-p), and the draw is a two-level prefix search.  Philox4x32-10 supplies one uniform per row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "launchers.h"

namespace ab {
namespace {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {  // ascending float order == ascending unsigned order
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  v = red[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Philox4x32-10: counter (c0..c3), key (k0, k1) -> first output word.
__device__ uint32_t philox_first(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
    c0 = n0, c1 = n1, c2 = n2, c3 = n3;
    k0 += 0x9E3779B9u, k1 += 0xBB67AE85u;
  }
  return c0;
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_rows_kernel(const T* __restrict__ logits, long long ld, float* __restrict__ work, const float* __restrict__ temps,
                   const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ penalty,
                   const long long* __restrict__ hist, const bool* __restrict__ hist_mask, int hist_len, int V,
                   int all_greedy, unsigned long long seed, unsigned long long offset, long long* __restrict__ out_tok,
                   float* __restrict__ out_logp) {
  __shared__ float red[32];
  __shared__ int h_cnt[256];
  __shared__ float h_mass[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_k;
  __shared__ float s_above;
  __shared__ int s_found;
  __shared__ float s_scan[SAMPLE_THREADS];
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* lg = logits + (long long)row * ld;
  float* w = work + (long long)row * V;

  if (all_greedy) {
    float best = -CUDART_INF_F;
    int best_i = V;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const float x = to_float(lg[i]);
      if (x > best) best = x, best_i = i;  // ascending i per thread: ties keep the lowest index
    }
    const float m = block_max(best, red);
    // lowest index among the maxima
    int cand = (best == m) ? best_i : V;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int red_i[32];
    __syncthreads();
    if ((tid & 31) == 0) red_i[tid >> 5] = cand;
    __syncthreads();
    cand = red_i[tid & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) z += __expf(to_float(lg[i]) - m);
    z = block_sum(z, red);
    if (tid == 0) {
      out_tok[row] = cand < V ? cand : 0;
      out_logp[row] = -__logf(z);  // x[argmax] - m = 0
    }
    return;
  }

  // ---- temperature, row maximum
  const float inv_t = 1.f / fmaxf(temps[row], 1e-8f);
  float mx = -CUDART_INF_F;
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    const float x = to_float(lg[i]) * inv_t;
    w[i] = x;
    mx = fmaxf(mx, x);
  }
  mx = block_max(mx, red);  // (the barriers inside also make every thread's w[] writes visible to the block)

  // ---- top-k: key of the k-th largest value by radix selection on counts
  uint32_t thr_key = 0;  // keep x iff order_key(x) >= thr_key
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < V) {
    if (tid == 0) s_prefix = 0, s_k = k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) h_cnt[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix, hi_mask = pass ? (0xffffffffu << (shift + 8)) : 0u;
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const uint32_t key = order_key(w[i]);
        if ((key & hi_mask) == prefix) atomicAdd(&h_cnt[(key >> shift) & 0xff], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int need = s_k, b = 255;
        for (; b > 0; --b) {
          if (h_cnt[b] >= need) break;
          need -= h_cnt[b];
        }
        s_k = need;
        s_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
    }
    thr_key = s_prefix;
  }

  // ---- top-p: key of the first token (descending) whose inclusive probability mass exceeds p
  const float p = top_p ? top_p[row] : 1.f;
  if (p < 1.f) {
    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const float x = w[i];
      if (order_key(x) >= thr_key) z += __expf(x - mx);
    }
    z = block_sum(z, red);
    const float target = p * z;
    if (tid == 0) s_prefix = 0, s_above = 0.f, s_found = 1;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) h_mass[tid] = 0.f;
      __syncthreads();
      const uint32_t prefix = s_prefix, hi_mask = pass ? (0xffffffffu << (shift + 8)) : 0u;
      for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = w[i];
        const uint32_t key = order_key(x);
        if (key >= thr_key && (key & hi_mask) == prefix) atomicAdd(&h_mass[(key >> shift) & 0xff], __expf(x - mx));
      }
      __syncthreads();
      if (tid == 0 && s_found) {
        float above = s_above;
        int b = 255;
        for (; b >= 0; --b) {
          if (above + h_mass[b] > target) break;
          above += h_mass[b];
        }
        if (b < 0) {
          s_found = 0;  // the mass never exceeds p * Z (rounding): keep everything
        } else {
          s_above = above;
          s_prefix = prefix | ((uint32_t)b << shift);
        }
      }
      __syncthreads();
    }
    if (s_found) thr_key = max(thr_key, s_prefix);
  }

  // ---- filtered values, frequency penalty
  const float pen = penalty ? penalty[row] : 0.f;
  if (thr_key != 0 || pen != 0.f) {
    for (int i = tid; i < V; i += SAMPLE_THREADS)
      if (order_key(w[i]) < thr_key) w[i] = -CUDART_INF_F;
    __syncthreads();
    if (pen != 0.f && hist != nullptr) {
      for (int j = tid; j < hist_len; j += SAMPLE_THREADS) {
        if (hist_mask && !hist_mask[(long long)row * hist_len + j]) continue;
        long long tok = hist[(long long)row * hist_len + j];
        tok = tok < 0 ? 0 : tok;
        if (tok < V) atomicAdd(&w[tok], -pen);
      }
      __syncthreads();
      mx = -CUDART_INF_F;
      for (int i = tid; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, w[i]);
      mx = block_max(mx, red);
    }
  }

  // ---- draw: per-thread contiguous chunks, block prefix over the chunk sums, walk the chunk that holds the target
  const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) mine += __expf(w[i] - mx);
  s_scan[tid] = mine;
  __syncthreads();
  for (int o = 1; o < SAMPLE_THREADS; o <<= 1) {  // inclusive Hillis-Steele scan
    const float add = tid >= o ? s_scan[tid - o] : 0.f;
    __syncthreads();
    s_scan[tid] += add;
    __syncthreads();
  }
  const float total = s_scan[SAMPLE_THREADS - 1];
  const uint32_t bits = philox_first((uint32_t)offset, (uint32_t)(offset >> 32), (uint32_t)row, 0u, (uint32_t)seed, (uint32_t)(seed >> 32));
  const float target = ((bits >> 8) + 0.5f) * (1.f / 16777216.f) * total;  // u in (0, 1)
  if (tid == 0) s_found = -1;
  __syncthreads();
  const float before = tid ? s_scan[tid - 1] : 0.f;  // intervals [before, s_scan[tid]) tile [0, total) without gaps
  const bool holder = mine > 0.f && target >= before && (target < s_scan[tid] || tid == SAMPLE_THREADS - 1);
  if (holder) {
    float run = before;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      const float e = __expf(w[i] - mx);
      if (e > 0.f) {
        pick = i;  // the last token with mass seen so far: the fallback when rounding leaves the target just above
        run += e;
        if (target < run) break;
      }
    }
    if (pick >= 0) atomicMax(&s_found, pick);
  }
  __syncthreads();
  if (s_found < 0 && tid == 0) {  // target fell past the last chunk with mass (rounding): take the maximum's index
    for (int i = 0; i < V; ++i)
      if (w[i] == mx) { s_found = i; break; }
  }
  __syncthreads();
  if (tid == 0) {
    const int tok = max(s_found, 0);
    out_tok[row] = tok;
    out_logp[row] = w[tok] - mx - __logf(total);
  }
}

}  // namespace

int sample_rows(const void* logits, bool is_bf16, long long ld, float* work, const float* temps, const int* top_k,
                const float* top_p, const float* penalty, const long long* hist, const bool* hist_mask, int hist_len,
                int rows, int V, bool all_greedy, unsigned long long seed, unsigned long long offset, long long* out_tok,
                float* out_logp, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (V <= 0 || temps == nullptr) return -1;
  if (is_bf16)
    sample_rows_kernel<__nv_bfloat16><<<rows, SAMPLE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld, work, temps, top_k, top_p, penalty,
                                                                     hist, hist_mask, hist_len, V, all_greedy ? 1 : 0, seed, offset,
                                                                     out_tok, out_logp);
  else
    sample_rows_kernel<float><<<rows, SAMPLE_THREADS, 0, st>>>((const float*)logits, ld, work, temps, top_k, top_p, penalty, hist,
                                                             hist_mask, hist_len, V, all_greedy ? 1 : 0, seed, offset, out_tok,
                                                             out_logp);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
