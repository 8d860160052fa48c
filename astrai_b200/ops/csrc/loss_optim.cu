// Cross-entropy over vocabulary rows (label smoothing, ignore_index, in-place gradient), token log-prob gather,
// fused AdamW on flat buffers, sum-of-squares and the clip coefficient.
// Reference semantics: F.cross_entropy on fp32 logits (astrai/trainer/strategy.py:336-340, :385-390),
// log_softmax + gather (strategy.py:66-70), clip_grad_norm + AdamW (astrai/parallel/executor.py:238-242).
#include "common.cuh"
#include "launchers.h"

namespace ab {

// One CTA per row of logits [rows, V] (row stride ld).
//   loss_row = lse - (1-eps)*z[y] - eps/V * sum_j z[j]        (0 for ignored rows)
//   if dlogits: dlogits[j] = gscale * (softmax_j - (1-eps)*[j==y] - eps/V), gscale = *grad_scale (device scalar)
// dlogits may alias logits.  Also emits logprob_row = z[y] - lse when `logprob` is given.
template <typename T>
__global__ void __launch_bounds__(512) ce_row_kernel(const T* __restrict__ logits, T* dlogits,
                                                     const long long* __restrict__ targets, float* __restrict__ loss,
                                                     float* __restrict__ logprob, const float* __restrict__ grad_scale,
                                                     int V, long long ld, float smoothing, long long ignore_index) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const T* z = logits + row * ld;
  const long long y = targets[row];
  const bool ignored = (y == ignore_index) || y < 0 || y >= V;
  const int nvec = V >> 3;
  const bool vec_ok = (V % 8 == 0) && (ld % 8 == 0);

  float m = -INFINITY, s = 0.f, zsum = 0.f;  // online max / sum-exp, plus plain sum for smoothing
  if (vec_ok) {
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      Vec8<T> v;
      v.load(z + c * 8);
      float f[8];
      v.unpack(f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc += __expf(f[j] - nm);
        zsum += f[j];
      }
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
  } else {
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
      const float f = to_f(z[c]);
      const float nm = fmaxf(m, f);
      s = s * __expf(m - nm) + __expf(f - nm);
      m = nm;
      zsum += f;
    }
  }
  const float gm = block_max(m, scratch);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum(s, scratch);
  zsum = block_sum(zsum, scratch);
  const float lse = gm + __logf(s);

  if (threadIdx.x == 0) {
    const float zy = ignored ? 0.f : to_f(z[y]);
    if (loss) loss[row] = ignored ? 0.f : (lse - (1.f - smoothing) * zy - smoothing * zsum / V);
    if (logprob) logprob[row] = ignored ? 0.f : (zy - lse);
  }
  if (dlogits == nullptr) return;
  __syncthreads();  // z[y] was read above; dlogits may alias logits
  const float gs = ignored ? 0.f : *grad_scale;
  const float inv = 1.f / s, off = smoothing / V;
  T* d = dlogits + row * ld;
  if (vec_ok) {
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      Vec8<T> v;
      v.load(z + c * 8);
      float f[8];
      v.unpack(f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = __expf(f[j] - gm) * inv - off;
        if ((long long)(c * 8 + j) == y) p -= (1.f - smoothing);
        f[j] = p * gs;
      }
      v.pack(f);
      v.store(d + c * 8);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
      float p = __expf(to_f(z[c]) - gm) * inv - off;
      if ((long long)c == y) p -= (1.f - smoothing);
      d[c] = from_f<T>(p * gs);
    }
  }
}

void ce_rows(const void* logits, void* dlogits, const long long* targets, float* loss, float* logprob,
             const float* grad_scale, long long rows, int V, long long ld, float smoothing, long long ignore_index,
             bool is_bf16, cudaStream_t st) {
  if (rows == 0) return;
  if (is_bf16)
    ce_row_kernel<__nv_bfloat16><<<rows, 512, 0, st>>>((const __nv_bfloat16*)logits, (__nv_bfloat16*)dlogits, targets,
                                                       loss, logprob, grad_scale, V, ld, smoothing, ignore_index);
  else
    ce_row_kernel<float><<<rows, 512, 0, st>>>((const float*)logits, (float*)dlogits, targets, loss, logprob,
                                                grad_scale, V, ld, smoothing, ignore_index);
}

// dlogits[j] = g_row * ([j==y] - softmax_j): backward of logprob_row = z[y] - lse.  May alias logits.
template <typename T>
__global__ void __launch_bounds__(512) logprob_bwd_kernel(const T* __restrict__ logits, T* dlogits,
                                                          const long long* __restrict__ targets,
                                                          const float* __restrict__ logprob,
                                                          const float* __restrict__ g_rows, int V, long long ld) {
  const long long row = blockIdx.x;
  const T* z = logits + row * ld;
  T* d = dlogits + row * ld;
  const long long y = targets[row];
  const bool bad = y < 0 || y >= V;
  // lse = z[y] - logprob
  __shared__ float lse_s;
  if (threadIdx.x == 0) lse_s = bad ? 0.f : to_f(z[y]) - logprob[row];
  __syncthreads();
  const float lse = lse_s, g = bad ? 0.f : g_rows[row];
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float p = -__expf(to_f(z[c]) - lse);
    if ((long long)c == y) p += 1.f;
    d[c] = from_f<T>(p * g);
  }
}

void logprob_bwd(const void* logits, void* dlogits, const long long* targets, const float* logprob,
                 const float* g_rows, long long rows, int V, long long ld, bool is_bf16, cudaStream_t st) {
  if (rows == 0) return;
  if (is_bf16)
    logprob_bwd_kernel<__nv_bfloat16><<<rows, 512, 0, st>>>((const __nv_bfloat16*)logits, (__nv_bfloat16*)dlogits,
                                                            targets, logprob, g_rows, V, ld);
  else
    logprob_bwd_kernel<float><<<rows, 512, 0, st>>>((const float*)logits, (float*)dlogits, targets, logprob, g_rows,
                                                    V, ld);
}

// ---------------------------------------------------------------- optimizer
// out[0] += sum(x^2).  Grid-stride, one atomic per CTA.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float f = to_f(x[i]);
    s += f * f;
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

void sumsq_accum(const void* x, long long n, float* out, bool is_bf16, cudaStream_t st) {
  if (n == 0) return;
  long long g = (n + 1023) / 1024;
  const int grid = (int)(g < 148 * 8 ? g : 148 * 8);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, n, out);
  else sumsq_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, out);
}

// coef[0] = min(1, max_norm / (sqrt(sumsq * pre_scale^2) + 1e-6)) * pre_scale ; norm_out[0] = sqrt(sumsq)*pre_scale.
// pre_scale folds an averaging factor (for example 1/world) into both the norm and the coefficient.
__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float pre_scale, float* coef, float* norm_out) {
  const float norm = sqrtf(sumsq[0]) * pre_scale;
  if (norm_out) norm_out[0] = norm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (norm + 1e-6f));
  coef[0] = c * pre_scale;
}

void clip_coef(const float* sumsq, float max_norm, float pre_scale, float* coef, float* norm_out, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, max_norm, pre_scale, coef, norm_out);
}

// Decoupled-weight-decay Adam on flat buffers.  g is fp32 (accumulated gradient), scaled by *gscale (device
// scalar, may be null).  `master` (fp32 copy of the weights) is optional; without it the bf16 weights are the state.
template <typename P>
__global__ void adamw_kernel(P* __restrict__ p, float* __restrict__ master, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2_sqrt, const float* __restrict__ gscale,
                             int zero_grad, float* g_mut) {
  const float gs = gscale ? *gscale : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float grad = g[i] * gs;
    float w = master ? master[i] : to_f(p[i]);
    const float mi = b1 * m[i] + (1.f - b1) * grad;
    const float vi = b2 * v[i] + (1.f - b2) * grad * grad;
    m[i] = mi;
    v[i] = vi;
    w *= (1.f - lr * wd);
    w -= (lr / bc1) * mi / (sqrtf(vi) / bc2_sqrt + eps);
    if (master) master[i] = w;
    p[i] = from_f<P>(w);
    if (zero_grad) g_mut[i] = 0.f;
  }
}

void adamw_step(void* p, float* master, float* g, float* m, float* v, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, const float* gscale, bool zero_grad, bool p_bf16, cudaStream_t st) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2_sqrt = sqrtf(1.f - powf(b2, (float)step));
  long long gsz = (n + 1023) / 1024;
  const int grid = (int)(gsz < 148 * 16 ? gsz : 148 * 16);
  if (p_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)p, master, g, m, v, n, lr, b1, b2, eps, wd, bc1,
                                                       bc2_sqrt, gscale, zero_grad ? 1 : 0, g);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>((float*)p, master, g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2_sqrt,
                                               gscale, zero_grad ? 1 : 0, g);
}

// dst(fp32) += alpha * src ; src may be bf16 or fp32.
template <typename T>
__global__ void axpy_f32_kernel(float* __restrict__ dst, const T* __restrict__ src, long long n, float alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] += alpha * to_f(src[i]);
}

void axpy_f32(float* dst, const void* src, long long n, float alpha, bool src_bf16, cudaStream_t st) {
  if (n == 0) return;
  long long gsz = (n + 1023) / 1024;
  const int grid = (int)(gsz < 148 * 16 ? gsz : 148 * 16);
  if (src_bf16) axpy_f32_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(dst, (const __nv_bfloat16*)src, n, alpha);
  else axpy_f32_kernel<float><<<grid, 256, 0, st>>>(dst, (const float*)src, n, alpha);
}

}  // namespace ab
