// Inference attention kernels over a slot-addressed (paged) KV pool.
//
//   kv_append     : scatter this step's K/V rows into the pool (slot = out_cache_loc[token]).
//   paged_decode  : flash-decoding.  One CTA per (kv head, request, KV split); the G query heads that share a kv
//                   head are processed together so every K/V byte is read once per split (GQA head packing).
//                   Partials (un-normalised O, running max, sum) go to a caller-provided scratch; the LAST CTA to
//                   finish a (request, kv head) merges its splits and writes bf16 output - no second launch.
// Replaces the reference's decode_split_kv_mma + decode_combine pair (csrc/kernels/attention/decode_split_kv_mma.cuh:20-183,
// decode_split_kv.cuh:115-144).  Decode is HBM-bound (~4 FLOP per KV byte), so the math stays on the CUDA cores and
// the kernel is shaped for bytes in flight: 16-byte loads, several tokens per warp iteration, unrolled.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "launchers.h"

namespace ab {

__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                 __nv_bfloat16* __restrict__ k_buf, __nv_bfloat16* __restrict__ v_buf,
                                 const int* __restrict__ loc, long long tokens, int row_elems, long long n_slots) {
  const int vec = row_elems >> 3;
  const long long total = tokens * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int c = (int)(i % vec) * 8;
    const long long slot = loc[t];
    if (slot < 0 || slot >= n_slots) continue;  // never write outside the pool
    *reinterpret_cast<uint4*>(k_buf + slot * row_elems + c) = *reinterpret_cast<const uint4*>(k_new + t * row_elems + c);
    *reinterpret_cast<uint4*>(v_buf + slot * row_elems + c) = *reinterpret_cast<const uint4*>(v_new + t * row_elems + c);
  }
}

void kv_append(const void* k_new, const void* v_new, void* k_buf, void* v_buf, const int* loc, long long tokens,
               int row_elems, long long n_slots, cudaStream_t st) {
  if (tokens == 0) return;
  const long long total = tokens * (row_elems / 8);
  const int grid = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  kv_append_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)k_buf,
                                         (__nv_bfloat16*)v_buf, loc, tokens, row_elems, n_slots);
}

constexpr int DEC_WARPS = 4;
constexpr int MAXG = 8;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// D = head dim (32/64/128/256).  LPT lanes cooperate on one token (8 dims each); a warp handles 32/LPT tokens at once.
template <int D, int GT>  // GT: query heads per kv head, 1..8 (compile-time, so the per-head state lives in registers)
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_buf,
                    const __nv_bfloat16* __restrict__ v_buf, const int* __restrict__ req_to_token,
                    const int* __restrict__ req_pool_indices, const long long* __restrict__ seq_lens,
                    float* __restrict__ o_part, float* __restrict__ ml_part, int* __restrict__ counters,
                    __nv_bfloat16* __restrict__ out, int n_q_heads, int n_kv_heads, int max_ctx, long long n_slots,
                    float scale, int max_splits, int table_rows, const __nv_bfloat16* __restrict__ k_new,
                    const __nv_bfloat16* __restrict__ v_new, __nv_bfloat16* __restrict__ k_pool_w,
                    __nv_bfloat16* __restrict__ v_pool_w) {
  constexpr int LPT = D / 8;
  constexpr int TPW = 32 / LPT;  // tokens per warp iteration
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
  constexpr int G = GT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPT, dl = lane % LPT;  // token sub-group inside the warp, dim chunk of this lane
  // Host-supplied metadata is not trusted: a length beyond the table row is cut to the row, a request row outside the
  // table (when the caller told us how many rows there are) attends to nothing.  Neither can read out of bounds.
  long long len = seq_lens[b];
  len = len < 0 ? 0 : (len > max_ctx ? (long long)max_ctx : len);
  int table_row = req_pool_indices[b];
  if (table_row < 0 || (table_rows > 0 && table_row >= table_rows)) table_row = 0, len = 0;
  const int* table = req_to_token + (long long)table_row * max_ctx;
  const long long chunk = ((len + splits - 1) / splits + 15) / 16 * 16;
  const long long t_begin = (long long)split * chunk;
  const long long t_end = t_begin + chunk < len ? t_begin + chunk : len;

  float qf[GT][8], acc[GT][8], m[GT], l[GT];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.f, qf[g][j] = 0.f;
    if (g < G) {
      load8(q + ((long long)b * n_q_heads + kvh * G + g) * D + dl * 8, qf[g]);
#pragma unroll
      for (int j = 0; j < 8; ++j) qf[g][j] *= scale;
    }
  }

  const long long row = (long long)n_kv_heads * D;
  // Fused append (k_new != null): this step's key / value row of the request is not in the pool yet.  Every CTA takes
  // the last position (len - 1) from k_new / v_new instead of the pool, so no CTA depends on another one's write, and
  // the CTA of split 0 also stores the row into the slot the table names for that position.
  const long long t_new = (k_new != nullptr) ? len - 1 : -1;
  const __nv_bfloat16* k_new_row = k_new ? k_new + ((long long)b * n_kv_heads + kvh) * D : nullptr;
  const __nv_bfloat16* v_new_row = v_new ? v_new + ((long long)b * n_kv_heads + kvh) * D : nullptr;
  if (k_new != nullptr && split == 0 && len > 0 && threadIdx.x < 2 * (D / 8)) {
    const long long slot = table[len - 1];
    if (slot >= 0 && slot < n_slots) {
      const int which = threadIdx.x / (D / 8), c = (threadIdx.x % (D / 8)) * 8;
      const __nv_bfloat16* src = which ? v_new_row : k_new_row;
      __nv_bfloat16* dst = (which ? v_pool_w : k_pool_w) + slot * row + (long long)kvh * D;
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
    }
  }
  // Each lane group takes UNR tokens per trip.  The loads of trip i + 1 (table entries, then K and V rows - two dependent
  // round trips to memory) are issued BEFORE the arithmetic of trip i, into a second register set, so the memory
  // latency of a trip hides behind the previous trip's math; within a trip the softmax state of a head is rescaled
  // once for the UNR tokens together, not once per token.
  constexpr int UNR = GT >= 7 ? 2 : 4;  // two register sets of UNR rows each: fewer rows when many heads share a lane
  const long long stride = (long long)DEC_WARPS * TPW * UNR;
  auto load_trip = [&](long long t0, uint4 (&kraw)[UNR], uint4 (&vraw)[UNR], bool (&live)[UNR]) {
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long t = t0 + (long long)u * TPW + sub;
      const bool valid = t < t_end;
      long long slot = valid ? (long long)table[t] : -1;
      live[u] = valid && slot >= 0 && slot < n_slots;  // a corrupt table entry must not fault: its score is masked
      if (!live[u]) slot = 0;
      if (t == t_new) {  // the token of this step: straight from the projection's output
        kraw[u] = *reinterpret_cast<const uint4*>(k_new_row + dl * 8);
        vraw[u] = *reinterpret_cast<const uint4*>(v_new_row + dl * 8);
      } else {
        kraw[u] = *reinterpret_cast<const uint4*>(k_buf + slot * row + (long long)kvh * D + dl * 8);
        vraw[u] = *reinterpret_cast<const uint4*>(v_buf + slot * row + (long long)kvh * D + dl * 8);
      }
    }
  };
  auto compute_trip = [&](const uint4 (&kraw)[UNR], const uint4 (&vraw)[UNR], const bool (&live)[UNR]) {
    float sc[GT][UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      float kf[8];
      const __nv_bfloat162* hk = reinterpret_cast<const __nv_bfloat162*>(&kraw[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(hk[i]);
        kf[2 * i] = a.x, kf[2 * i + 1] = a.y;
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += qf[g][j] * kf[j];
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        sc[g][u] = live[u] ? s : -INFINITY;
      }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float mx = sc[g][0];
#pragma unroll
      for (int u = 1; u < UNR; ++u) mx = fmaxf(mx, sc[g][u]);
      const float nm = fmaxf(m[g], mx);
      const float alpha = (nm == -INFINITY) ? 1.f : __expf(m[g] - nm);
      l[g] *= alpha;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[g][j] *= alpha;
#pragma unroll
      for (int u = 0; u < UNR; ++u) sc[g][u] = (nm == -INFINITY) ? 0.f : __expf(sc[g][u] - nm);  // now the probabilities
      m[g] = nm;
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      float vf[8];
      const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&vraw[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 c = __bfloat1622float2(hv[i]);
        vf[2 * i] = c.x, vf[2 * i + 1] = c.y;
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        l[g] += sc[g][u];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(sc[g][u], vf[j], acc[g][j]);
      }
    }
  };
  {
    uint4 k_a[UNR], v_a[UNR], k_b[UNR], v_b[UNR];
    bool live_a[UNR], live_b[UNR];
    long long t0 = t_begin + (long long)warp * TPW * UNR;
    if (t0 < t_end) load_trip(t0, k_a, v_a, live_a);
    for (; t0 < t_end; t0 += 2 * stride) {
      const long long t1 = t0 + stride;
      const bool second = t1 < t_end;
      if (second) load_trip(t1, k_b, v_b, live_b);
      compute_trip(k_a, v_a, live_a);
      if (second) {
        if (t1 + stride < t_end) load_trip(t1 + stride, k_a, v_a, live_a);
        compute_trip(k_b, v_b, live_b);
      }
    }
  }

  // merge the TPW token sub-groups of the warp (same dims live LPT lanes apart)
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (g < G) {
#pragma unroll
      for (int o = LPT; o < 32; o <<= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m[g], o);
        const float ol = __shfl_xor_sync(0xffffffffu, l[g], o);
        const float nm = fmaxf(m[g], om);
        const float a = (nm == -INFINITY) ? 1.f : __expf(m[g] - nm);
        const float bsc = (nm == -INFINITY) ? 1.f : __expf(om - nm);
        l[g] = l[g] * a + ol * bsc;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float oa = __shfl_xor_sync(0xffffffffu, acc[g][j], o);
          acc[g][j] = acc[g][j] * a + oa * bsc;
        }
        m[g] = nm;
      }
    }
  }

  // merge the warps through shared memory
  __shared__ float s_acc[DEC_WARPS][GT][D];
  __shared__ float s_ml[DEC_WARPS][GT][2];
  __shared__ int s_last;
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g) {  // compile-time trip count: the per-head arrays must stay in registers
      if (g < G) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s_acc[warp][g][dl * 8 + j] = acc[g][j];
        if (dl == 0) s_ml[warp][g][0] = m[g], s_ml[warp][g][1] = l[g];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, s_ml[w][g][0]);
    float o = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float sc = (mm == -INFINITY) ? 0.f : __expf(s_ml[w][g][0] - mm);
      o += s_acc[w][g][d] * sc;
      ll += s_ml[w][g][1] * sc;
    }
    const long long head = (long long)b * n_q_heads + kvh * G + g;
    o_part[(head * max_splits + split) * D + d] = o;
    if (d == 0) {
      ml_part[(head * max_splits + split) * 2] = mm;
      ml_part[(head * max_splits + split) * 2 + 1] = ll;
    }
  }

  // the last CTA of this (request, kv head) combines the splits
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&counters[b * n_kv_heads + kvh], 1);
    s_last = (done == splits - 1);
    if (s_last) counters[b * n_kv_heads + kvh] = 0;  // ready for the next launch (graph replay included)
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const long long head = (long long)b * n_q_heads + kvh * G + g;
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, ml_part[(head * max_splits + s) * 2]);
    float o = 0.f, ll = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float sc = (mm == -INFINITY) ? 0.f : __expf(ml_part[(head * max_splits + s) * 2] - mm);
      o += o_part[(head * max_splits + s) * D + d] * sc;
      ll += ml_part[(head * max_splits + s) * 2 + 1] * sc;
    }
    out[head * D + d] = __float2bfloat16_rn(ll > 0.f ? o / ll : 0.f);
  }
}

int paged_decode_splits(int batch, int n_kv_heads, long long max_len, int max_splits) {
  const long long base = (long long)batch * n_kv_heads;
  long long s = (148 * 2) / base;                // two CTAs fit on an SM (register use): aim for one full wave
  const long long by_len = (max_len + 127) / 128;  // at least 128 tokens per split
  if (s > by_len) s = by_len;
  if (s > max_splits) s = max_splits;
  return (int)(s < 1 ? 1 : s);
}

int paged_decode(const void* q, const void* k_buf, const void* v_buf, const int* req_to_token,
                 const int* req_pool_indices, const long long* seq_lens, float* o_part, float* ml_part, int* counters,
                 void* out, int batch, int n_q_heads, int n_kv_heads, int head_dim, int max_ctx, long long n_slots,
                 float scale, int splits, int max_splits, int table_rows, cudaStream_t st, const void* k_new,
                 const void* v_new) {
  if (batch == 0) return 0;
  if ((k_new == nullptr) != (v_new == nullptr)) return -6;
  if (n_q_heads % n_kv_heads || n_q_heads / n_kv_heads > MAXG) return -1;
  if (splits < 1 || splits > max_splits) return -2;
  const dim3 grid(n_kv_heads, batch, splits), block(DEC_WARPS * 32);
  const int G = n_q_heads / n_kv_heads;
  const int gt = G;  // one instantiation per group size: the per-head loops unroll without predicates
#define AB_DEC(DD, GG)                                                                                               \
  paged_decode_kernel<DD, GG><<<grid, block, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_buf,          \
                                                      (const __nv_bfloat16*)v_buf, req_to_token, req_pool_indices,   \
                                                      seq_lens, o_part, ml_part, counters, (__nv_bfloat16*)out,      \
                                                      n_q_heads, n_kv_heads, max_ctx, n_slots, scale, max_splits, table_rows, \
                                                      (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new,     \
                                                      (__nv_bfloat16*)const_cast<void*>(k_buf),                     \
                                                      (__nv_bfloat16*)const_cast<void*>(v_buf))
#define AB_DEC_G(DD)                 \
  switch (gt) {                      \
    case 1: AB_DEC(DD, 1); break;    \
    case 2: AB_DEC(DD, 2); break;    \
    case 3: AB_DEC(DD, 3); break;    \
    case 4: AB_DEC(DD, 4); break;    \
    case 5: AB_DEC(DD, 5); break;    \
    case 6: AB_DEC(DD, 6); break;    \
    case 7: AB_DEC(DD, 7); break;    \
    default: AB_DEC(DD, 8); break;   \
  }
  switch (head_dim) {
    case 32: AB_DEC_G(32); break;
    case 64: AB_DEC_G(64); break;
    case 128: AB_DEC_G(128); break;
    case 256: AB_DEC_G(256); break;
    default: return -3;
  }
#undef AB_DEC_G
#undef AB_DEC
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
