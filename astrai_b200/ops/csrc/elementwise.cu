// RMSNorm, rotary embedding, SwiGLU and embedding kernels (forward and backward).
// All are HBM-bound: 16-byte vector I/O, fp32 math, one pass over the data where possible.
// Reference behaviour: F.rms_norm (astrai/model/components/norm.py:15), interleaved-pair RoPE
// (csrc/kernels/rotary/rotary_emb.cu:27-41), up*silu(gate) (astrai/model/components/mlp.py:41).
#include "common.cuh"
#include "launchers.h"

namespace ab {

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w.  One CTA per row, the row held in registers.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                          T* __restrict__ y, float* __restrict__ rstd_out,
                                                          int cols, float eps, const T* __restrict__ res,
                                                          T* __restrict__ xsum) {
  // With `res` the row normalised is x + res, rounded to T and also written to `xsum` (residual add fused in).
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  const int nvec = cols >> 3;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      Vec8<T> t;
      t.load(xr + c * 8);
      t.unpack(v[i]);
      if (res != nullptr) {
        Vec8<T> rv;
        float rf[8];
        rv.load(res + row * cols + c * 8);
        rv.unpack(rf);
#pragma unroll
        for (int j = 0; j < 8; ++j) rf[j] += v[i][j];
        rv.pack(rf);
        rv.store(xsum + row * cols + c * 8);
        rv.unpack(v[i]);  // the rounded sum is what the unfused path would normalise
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / cols + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      Vec8<T> wv;
      wv.load(w + c * 8);
      float wf[8], o[8];
      wv.unpack(wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wf[j];
      Vec8<T> ov;
      ov.pack(o);
      ov.store(yr + c * 8);
    }
  }
}

// Any width: one warp per row, scalar accesses (per-head q/k norms, odd sizes).
template <typename T>
__global__ void rmsnorm_fwd_small_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                         float* __restrict__ rstd_out, long long rows, int cols, float eps) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + row * cols;
  float ss = 0.f;
  for (int c = lane; c < cols; c += 32) {
    float f = to_f(xr[c]);
    ss += f * f;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / cols + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
  for (int c = lane; c < cols; c += 32) y[row * cols + c] = from_f<T>(to_f(xr[c]) * rstd * to_f(w[c]));
}

// dx = rstd * (g*w) - x * rstd^3 * mean(g*w*x);  dw partial = sum_rows g * x * rstd.
// Persistent CTAs walk rows; each thread owns fixed columns, so dw partials stay in registers.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                                          const T* __restrict__ w, const float* __restrict__ rstd,
                                                          T* __restrict__ dx, float* __restrict__ dw_partial,
                                                          long long rows, int cols, const T* __restrict__ gres) {
  // With `gres` the gradient that reaches x along the residual branch is added into dx here.
  __shared__ float scratch[32];
  const int nvec = cols >> 3;
  float wf[VPT][8], acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f, wf[i][j] = 0.f;
    if (c < nvec) {
      Vec8<T> wv;
      wv.load(w + c * 8);
      wv.unpack(wf[i]);
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float r = rstd[row];
    float xv[VPT][8], gv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nvec) {
        Vec8<T> a, b;
        a.load(x + row * cols + c * 8);
        b.load(g + row * cols + c * 8);
        a.unpack(xv[i]);
        b.unpack(gv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += gv[i][j] * wf[i][j] * xv[i][j];
          acc[i][j] += gv[i][j] * xv[i][j] * r;
        }
      }
    }
    dot = block_sum(dot, scratch);
    const float k = dot * r * r * r / cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gv[i][j] * wf[i][j] * r - xv[i][j] * k;
        if (gres != nullptr) {
          Vec8<T> rv;
          float rf[8];
          rv.load(gres + row * cols + c * 8);
          rv.unpack(rf);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rf[j];
        }
        Vec8<T> ov;
        ov.pack(o);
        ov.store(dx + row * cols + c * 8);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) dw_partial[(long long)blockIdx.x * cols + c * 8 + j] = acc[i][j];
    }
  }
}

template <typename T>
__global__ void rmsnorm_bwd_small_kernel(const T* __restrict__ g, const T* __restrict__ x, const T* __restrict__ w,
                                         const float* __restrict__ rstd, T* __restrict__ dx,
                                         float* __restrict__ dw_accum, long long rows, int cols) {
  // One warp per row; dw goes through fp32 atomics (small widths only).
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float r = rstd[row];
  float dot = 0.f;
  for (int c = lane; c < cols; c += 32) dot += to_f(g[row * cols + c]) * to_f(w[c]) * to_f(x[row * cols + c]);
  dot = warp_sum(dot);
  const float k = dot * r * r * r / cols;
  for (int c = lane; c < cols; c += 32) {
    const float gf = to_f(g[row * cols + c]), xf = to_f(x[row * cols + c]);
    dx[row * cols + c] = from_f<T>(gf * to_f(w[c]) * r - xf * k);
    atomicAdd(dw_accum + c, gf * xf * r);
  }
}

// out[c] = sum_p partial[p, c].  Block (32, 8): 32 adjacent columns, 8 row-lanes striding over the parts.
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts, int cols) {
  __shared__ float acc[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols)
    for (int p = threadIdx.y; p < parts; p += 8) s += partial[(long long)p * cols + c];
  acc[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += acc[j][threadIdx.x];
    out[c] = t;
  }
}

template <typename T>
static void rmsnorm_fwd_t(const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                          cudaStream_t st, const void* res, void* xsum) {
  if (rows == 0) return;
  if (cols % 8 == 0 && cols >= 512 && cols <= 16384) {
    const int nvec = cols / 8;
    auto X = (const T*)x; auto W = (const T*)w; auto Y = (T*)y; auto R = (const T*)res; auto XS = (T*)xsum;
    if (nvec <= 256) rmsnorm_fwd_kernel<T, 1><<<rows, 256, 0, st>>>(X, W, Y, rstd, cols, eps, R, XS);
    else if (nvec <= 512) rmsnorm_fwd_kernel<T, 2><<<rows, 256, 0, st>>>(X, W, Y, rstd, cols, eps, R, XS);
    else if (nvec <= 1024) rmsnorm_fwd_kernel<T, 4><<<rows, 256, 0, st>>>(X, W, Y, rstd, cols, eps, R, XS);
    else rmsnorm_fwd_kernel<T, 8><<<rows, 256, 0, st>>>(X, W, Y, rstd, cols, eps, R, XS);
  } else {
    const int wpb = 8;
    rmsnorm_fwd_small_kernel<T><<<ceil_div(rows, wpb), wpb * 32, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd,
                                                                          rows, cols, eps);
  }
}

void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                 bool is_bf16, cudaStream_t st, const void* res, void* xsum) {
  if (is_bf16) rmsnorm_fwd_t<__nv_bfloat16>(x, w, y, rstd, rows, cols, eps, st, res, xsum);
  else rmsnorm_fwd_t<float>(x, w, y, rstd, rows, cols, eps, st, res, xsum);
}

bool rmsnorm_wide(int cols) { return cols % 8 == 0 && cols >= 512 && cols <= 16384; }

int rmsnorm_bwd_parts(long long rows, int cols) {
  // one row at a time per 256-thread block with a block-wide reduction in between: four blocks per SM keep enough
  // loads in flight to cover that latency
  if (cols % 8 == 0 && cols >= 512 && cols <= 16384) return (int)(rows < 592 ? rows : 592);  // 148 SMs x 4
  return 0;  // small path accumulates with atomics into a zeroed dw
}

template <typename T>
static void rmsnorm_bwd_t(const void* g, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                          float* partial, long long rows, int cols, cudaStream_t st, const void* gres) {
  if (rows == 0) return;
  const int parts = rmsnorm_bwd_parts(rows, cols);
  if (parts > 0) {
    const int nvec = cols / 8;
    auto G = (const T*)g; auto X = (const T*)x; auto W = (const T*)w; auto DX = (T*)dx; auto GR = (const T*)gres;
    if (nvec <= 256) rmsnorm_bwd_kernel<T, 1><<<parts, 256, 0, st>>>(G, X, W, rstd, DX, partial, rows, cols, GR);
    else if (nvec <= 512) rmsnorm_bwd_kernel<T, 2><<<parts, 256, 0, st>>>(G, X, W, rstd, DX, partial, rows, cols, GR);
    else if (nvec <= 1024) rmsnorm_bwd_kernel<T, 4><<<parts, 256, 0, st>>>(G, X, W, rstd, DX, partial, rows, cols, GR);
    else rmsnorm_bwd_kernel<T, 8><<<parts, 256, 0, st>>>(G, X, W, rstd, DX, partial, rows, cols, GR);
    colsum_kernel<<<ceil_div(cols, 32), dim3(32, 8), 0, st>>>(partial, dw, parts, cols);
  } else {
    cudaMemsetAsync(dw, 0, sizeof(float) * cols, st);
    const int wpb = 8;
    rmsnorm_bwd_small_kernel<T><<<ceil_div(rows, wpb), wpb * 32, 0, st>>>((const T*)g, (const T*)x, (const T*)w, rstd,
                                                                          (T*)dx, dw, rows, cols);
  }
}

void rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, void* dx, float* dw, float* partial,
                 long long rows, int cols, bool is_bf16, cudaStream_t st, const void* gres) {
  if (is_bf16) rmsnorm_bwd_t<__nv_bfloat16>(g, x, w, rstd, dx, dw, partial, rows, cols, st, gres);
  else rmsnorm_bwd_t<float>(g, x, w, rstd, dx, dw, partial, rows, cols, st, gres);
}

// ---------------------------------------------------------------- RoPE
// (x[2i], x[2i+1]) -> (x0*c - x1*s, x0*s + x1*c); `sign` = -1 gives the inverse rotation (backward).
// x is addressed as token*tok_stride + head*head_stride + d; the table row of a token is freqs + token*rot_dim
// floats laid out [rot_dim/2][cos, sin].  In place when out == x.
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ freqs,
                            long long tokens, int heads, int rot_dim, long long x_tok_stride, int x_head_stride,
                            long long o_tok_stride, int o_head_stride, float sign) {
  const int vec_per_head = rot_dim >> 3;
  const long long total = tokens * heads * vec_per_head;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    Vec8<T> in;
    in.load(x + t * x_tok_stride + (long long)h * x_head_stride + v * 8);
    float f[8], o[8];
    in.unpack(f);
    const float4* fr = reinterpret_cast<const float4*>(freqs + t * rot_dim + v * 8);
    const float4 cs0 = fr[0], cs1 = fr[1];  // (c0,s0,c1,s1), (c2,s2,c3,s3)
    const float c[4] = {cs0.x, cs0.z, cs1.x, cs1.z};
    const float s[4] = {cs0.y * sign, cs0.w * sign, cs1.y * sign, cs1.w * sign};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      o[2 * p] = f[2 * p] * c[p] - f[2 * p + 1] * s[p];
      o[2 * p + 1] = f[2 * p] * s[p] + f[2 * p + 1] * c[p];
    }
    Vec8<T> ov;
    ov.pack(o);
    ov.store(out + t * o_tok_stride + (long long)h * o_head_stride + v * 8);
  }
}

void rope_apply(const void* x, void* out, const float* freqs, long long tokens, int heads, int rot_dim,
                long long x_tok_stride, int x_head_stride, long long o_tok_stride, int o_head_stride, bool inverse,
                bool is_bf16, cudaStream_t st) {
  const long long total = tokens * heads * (rot_dim / 8);
  if (total == 0) return;
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  const float sign = inverse ? -1.f : 1.f;
  if (is_bf16)
    rope_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, freqs, tokens,
                                                      heads, rot_dim, x_tok_stride, x_head_stride, o_tok_stride,
                                                      o_head_stride, sign);
  else
    rope_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (float*)out, freqs, tokens, heads, rot_dim,
                                              x_tok_stride, x_head_stride, o_tok_stride, o_head_stride, sign);
}

// ---------------------------------------------------------------- SwiGLU
// y = up * silu(gate).  gate/up may be column halves of one [rows, 2F] tensor (in_stride = 2F).
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y,
                                  long long rows, int f, long long in_stride) {
  const int vec = f >> 3;
  const long long total = rows * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec;
    const int c = (int)(i % vec) * 8;
    Vec8<T> gv, uv, ov;
    gv.load(gate + r * in_stride + c);
    uv.load(up + r * in_stride + c);
    float g[8], u[8], o[8];
    gv.unpack(g);
    uv.unpack(u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = u[j] * g[j] / (1.f + __expf(-g[j]));
    ov.pack(o);
    ov.store(y + r * f + c);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ gate, const T* __restrict__ up,
                                  T* __restrict__ dgate, T* __restrict__ dup, long long rows, int f,
                                  long long in_stride, long long out_stride) {
  const int vec = f >> 3;
  const long long total = rows * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec;
    const int c = (int)(i % vec) * 8;
    Vec8<T> dv, gv, uv, og, ou;
    dv.load(dy + r * f + c);
    gv.load(gate + r * in_stride + c);
    uv.load(up + r * in_stride + c);
    float d[8], g[8], u[8], a[8], b[8];
    dv.unpack(d);
    gv.unpack(g);
    uv.unpack(u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sig;
      a[j] = d[j] * u[j] * (sig + silu * (1.f - sig));
      b[j] = d[j] * silu;
    }
    og.pack(a);
    ou.pack(b);
    og.store(dgate + r * out_stride + c);
    ou.store(dup + r * out_stride + c);
  }
}

static int ew_grid(long long total) {
  long long g = (total + 255) / 256;
  return (int)(g < 148 * 16 ? (g > 0 ? g : 1) : 148 * 16);
}

void swiglu_fwd(const void* gate, const void* up, void* y, long long rows, int f, long long in_stride, bool is_bf16,
                cudaStream_t st) {
  if (rows == 0) return;
  const int grid = ew_grid(rows * (f / 8));
  if (is_bf16)
    swiglu_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                            (__nv_bfloat16*)y, rows, f, in_stride);
  else
    swiglu_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)gate, (const float*)up, (float*)y, rows, f,
                                                    in_stride);
}

void swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup, long long rows, int f,
                long long in_stride, long long out_stride, bool is_bf16, cudaStream_t st) {
  if (rows == 0) return;
  const int grid = ew_grid(rows * (f / 8));
  if (is_bf16)
    swiglu_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)dgate,
        (__nv_bfloat16*)dup, rows, f, in_stride, out_stride);
  else
    swiglu_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)dy, (const float*)gate, (const float*)up,
                                                    (float*)dgate, (float*)dup, rows, f, in_stride, out_stride);
}

// ---------------------------------------------------------------- Embedding
template <typename T>
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const T* __restrict__ table,
                                     T* __restrict__ out, long long tokens, int dim, long long vocab) {
  const int vec = dim >> 3;
  const long long total = tokens * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int c = (int)(i % vec) * 8;
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // clamp instead of faulting on a bad id
    Vec8<T> v;
    v.load(table + id * dim + c);
    v.store(out + t * dim + c);
  }
}

// grad_table[ids[t]] += g[t]  (fp32 accumulation buffer)
template <typename T>
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const T* __restrict__ g,
                                     float* __restrict__ grad_table, long long tokens, int dim, long long vocab) {
  const long long total = tokens * dim;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dim;
    const int c = (int)(i % dim);
    const long long id = ids[t];
    if (id >= 0 && id < vocab) atomicAdd(grad_table + id * dim + c, to_f(g[i]));
  }
}

// Deterministic form: `sorted` are the token ids in ascending order and `perm[j]` the position in the batch of sorted
// entry j.  One CTA per sorted position; the CTA at the head of a run of equal ids sums that run's gradient rows in run
// order (a fixed order, whatever the scheduling) and adds the sum to the id's row - no atomics, no two CTAs per row.
template <typename T>
__global__ void embedding_bwd_sorted_kernel(const long long* __restrict__ sorted, const long long* __restrict__ perm,
                                            const T* __restrict__ g, float* __restrict__ grad_table, long long tokens,
                                            int dim, long long vocab) {
  const long long i = blockIdx.x;
  const long long id = sorted[i];
  if (id < 0 || id >= vocab) return;
  if (i > 0 && sorted[i - 1] == id) return;  // not the head of its run
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float acc = 0.f;
    for (long long j = i; j < tokens && sorted[j] == id; ++j) acc += to_f(g[perm[j] * dim + c]);
    grad_table[id * dim + c] += acc;
  }
}

void embedding_bwd_sorted(const long long* sorted, const long long* perm, const void* g, float* grad_table, long long tokens,
                          int dim, long long vocab, bool is_bf16, cudaStream_t st) {
  if (tokens == 0) return;
  const int threads = dim >= 256 ? 256 : 64;
  if (is_bf16)
    embedding_bwd_sorted_kernel<__nv_bfloat16><<<(unsigned)tokens, threads, 0, st>>>(sorted, perm, (const __nv_bfloat16*)g,
                                                                                      grad_table, tokens, dim, vocab);
  else
    embedding_bwd_sorted_kernel<float><<<(unsigned)tokens, threads, 0, st>>>(sorted, perm, (const float*)g, grad_table, tokens,
                                                                              dim, vocab);
}

void embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int dim, long long vocab,
                   bool is_bf16, cudaStream_t st) {
  if (tokens == 0) return;
  const int grid = ew_grid(tokens * (dim / 8));
  if (is_bf16)
    embedding_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out,
                                                               tokens, dim, vocab);
  else
    embedding_fwd_kernel<float><<<grid, 256, 0, st>>>(ids, (const float*)table, (float*)out, tokens, dim, vocab);
}

void embedding_bwd(const long long* ids, const void* g, float* grad_table, long long tokens, int dim, long long vocab,
                   bool is_bf16, cudaStream_t st) {
  if (tokens == 0) return;
  const int grid = ew_grid(tokens * dim);
  if (is_bf16)
    embedding_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)g, grad_table, tokens, dim,
                                                               vocab);
  else
    embedding_bwd_kernel<float><<<grid, 256, 0, st>>>(ids, (const float*)g, grad_table, tokens, dim, vocab);
}

}  // namespace ab
