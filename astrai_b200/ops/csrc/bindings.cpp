// torch.ops.astrai_b200.* : tensor-level entry points of the sm_100a kernels.
// Only this file sees torch headers; kernels live in torch-free .cu files (launchers.h).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <atomic>
#include <map>

#include "launchers.h"

namespace {

using at::Tensor;

// Number of kernels of this library launched by this process (each binding adds what it launches).
std::atomic<long long> g_launches{0};
inline void count(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count() { return g_launches.load(); }

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline bool is_bf16(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, "expected bf16 or fp32 tensor");
  return t.scalar_type() == at::kBFloat16;
}
#define CHECK_CUDA_CONTIG(t) TORCH_CHECK((t).is_cuda() && (t).is_contiguous(), #t " must be a contiguous CUDA tensor")

std::tuple<Tensor, Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(w);
  TORCH_CHECK(x.scalar_type() == w.scalar_type(), "rmsnorm: x and weight dtypes differ");
  const c10::cuda::CUDAGuard guard(x.device());
  const int cols = (int)x.size(-1);
  const long long rows = x.numel() / cols;
  Tensor y = at::empty_like(x);
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  count();
  ab::rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, cols, (float)eps,
                  is_bf16(x), stream());
  return {y, rstd};
}

std::tuple<Tensor, Tensor> rmsnorm_bwd(const Tensor& g, const Tensor& x, const Tensor& w, const Tensor& rstd) {
  CHECK_CUDA_CONTIG(g);
  CHECK_CUDA_CONTIG(x);
  const c10::cuda::CUDAGuard guard(x.device());
  const int cols = (int)x.size(-1);
  const long long rows = x.numel() / cols;
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty({cols}, x.options().dtype(at::kFloat));
  const int parts = ab::rmsnorm_bwd_parts(rows, cols);
  Tensor partial = at::empty({parts > 0 ? parts : 1, cols}, dw.options());
  count(2);
  ab::rmsnorm_bwd(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                  dw.data_ptr<float>(), partial.data_ptr<float>(), rows, cols, is_bf16(x), stream());
  return {dx, dw};
}

// Residual add fused into the norm: returns (x + res, rmsnorm(x + res) * w, rstd).  Wide rows only.
std::tuple<Tensor, Tensor, Tensor> add_rmsnorm_fwd(const Tensor& x, const Tensor& res, const Tensor& w, double eps) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(res);
  CHECK_CUDA_CONTIG(w);
  TORCH_CHECK(x.scalar_type() == w.scalar_type() && x.scalar_type() == res.scalar_type() && x.sizes() == res.sizes(),
              "add_rmsnorm: x, res and weight must agree in dtype, x and res in shape");
  const int cols = (int)x.size(-1);
  TORCH_CHECK(ab::rmsnorm_wide(cols), "add_rmsnorm: row width must be a multiple of 8 in [512, 16384]");
  const c10::cuda::CUDAGuard guard(x.device());
  const long long rows = x.numel() / cols;
  Tensor xsum = at::empty_like(x), y = at::empty_like(x);
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  count();
  ab::rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, cols, (float)eps, is_bf16(x),
                  stream(), res.data_ptr(), xsum.data_ptr());
  return {xsum, y, rstd};
}

// Backward of the fused form: dx = rmsnorm_bwd(g, x, w, rstd) + gres.
std::tuple<Tensor, Tensor> rmsnorm_bwd_add(const Tensor& g, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                           const Tensor& gres) {
  CHECK_CUDA_CONTIG(g);
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(gres);
  TORCH_CHECK(gres.scalar_type() == x.scalar_type() && gres.sizes() == x.sizes(), "rmsnorm_bwd_add: gres must match x");
  const int cols = (int)x.size(-1);
  TORCH_CHECK(ab::rmsnorm_wide(cols), "rmsnorm_bwd_add: row width must be a multiple of 8 in [512, 16384]");
  const c10::cuda::CUDAGuard guard(x.device());
  const long long rows = x.numel() / cols;
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty({cols}, x.options().dtype(at::kFloat));
  const int parts = ab::rmsnorm_bwd_parts(rows, cols);
  Tensor partial = at::empty({parts > 0 ? parts : 1, cols}, dw.options());
  count(2);
  ab::rmsnorm_bwd(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dw.data_ptr<float>(),
                  partial.data_ptr<float>(), rows, cols, is_bf16(x), stream(), gres.data_ptr());
  return {dx, dw};
}

// x, out: [tokens, heads, rot_dim] views with unit last stride; freqs: [tokens, rot_dim/2, 2] fp32 contiguous.
void rope(const Tensor& x, Tensor& out, const Tensor& freqs, bool inverse) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && out.dim() == 3 && x.stride(2) == 1 && out.stride(2) == 1, "rope: bad layout");
  TORCH_CHECK(freqs.is_contiguous() && freqs.scalar_type() == at::kFloat, "rope: freqs must be contiguous fp32");
  TORCH_CHECK(x.size(2) % 8 == 0 && freqs.numel() == x.size(0) * x.size(2), "rope: rot_dim must be a multiple of 8 and match freqs");
  TORCH_CHECK(x.stride(0) % 8 == 0 && x.stride(1) % 8 == 0 && out.stride(0) % 8 == 0 && out.stride(1) % 8 == 0 &&
                  (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0,
              "rope: views must keep 16-byte alignment");
  TORCH_CHECK(x.scalar_type() == out.scalar_type(), "rope: dtype mismatch");
  const c10::cuda::CUDAGuard guard(x.device());
  count();
  ab::rope_apply(x.data_ptr(), out.data_ptr(), freqs.data_ptr<float>(), x.size(0), (int)x.size(1), (int)x.size(2),
                 x.stride(0), (int)x.stride(1), out.stride(0), (int)out.stride(1), inverse, is_bf16(x), stream());
}

// gate, up: [rows, F] views sharing one row stride (for example the two halves of a [rows, 2F] GEMM output).
Tensor swiglu_fwd(const Tensor& gate, const Tensor& up) {
  TORCH_CHECK(gate.is_cuda() && gate.dim() == 2 && gate.stride(1) == 1 && up.stride(1) == 1 &&
                  gate.stride(0) == up.stride(0) && gate.size(1) % 8 == 0 && gate.stride(0) % 8 == 0,
              "swiglu: bad layout");
  const c10::cuda::CUDAGuard guard(gate.device());
  Tensor y = at::empty({gate.size(0), gate.size(1)}, gate.options());
  count();
  ab::swiglu_fwd(gate.data_ptr(), up.data_ptr(), y.data_ptr(), gate.size(0), (int)gate.size(1), gate.stride(0),
                 is_bf16(gate), stream());
  return y;
}

// returns [rows, 2F]: columns [0,F) = d gate, [F,2F) = d up
Tensor swiglu_bwd(const Tensor& dy, const Tensor& gate, const Tensor& up) {
  CHECK_CUDA_CONTIG(dy);
  const c10::cuda::CUDAGuard guard(gate.device());
  const long long rows = gate.size(0);
  const int f = (int)gate.size(1);
  Tensor d = at::empty({rows, 2 * (long long)f}, gate.options());
  char* base = static_cast<char*>(d.data_ptr());
  count();
  ab::swiglu_bwd(dy.data_ptr(), gate.data_ptr(), up.data_ptr(), base, base + (size_t)f * d.element_size(), rows, f,
                 gate.stride(0), 2LL * f, is_bf16(gate), stream());
  return d;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& table) {
  CHECK_CUDA_CONTIG(ids);
  CHECK_CUDA_CONTIG(table);
  TORCH_CHECK(ids.scalar_type() == at::kLong && table.size(1) % 8 == 0, "embedding: ids int64, dim % 8 == 0");
  const c10::cuda::CUDAGuard guard(table.device());
  auto shape = ids.sizes().vec();
  shape.push_back(table.size(1));
  Tensor out = at::empty(shape, table.options());
  count();
  ab::embedding_fwd(ids.data_ptr<int64_t>() ? (const long long*)ids.data_ptr<int64_t>() : nullptr, table.data_ptr(),
                    out.data_ptr(), ids.numel(), (int)table.size(1), table.size(0), is_bf16(table), stream());
  return out;
}

void embedding_bwd_(const Tensor& ids, const Tensor& g, Tensor& grad_table) {
  CHECK_CUDA_CONTIG(ids);
  CHECK_CUDA_CONTIG(g);
  CHECK_CUDA_CONTIG(grad_table);
  TORCH_CHECK(grad_table.scalar_type() == at::kFloat, "embedding_bwd_: fp32 accumulation buffer expected");
  const c10::cuda::CUDAGuard guard(g.device());
  count();
  ab::embedding_bwd((const long long*)ids.data_ptr<int64_t>(), g.data_ptr(), grad_table.data_ptr<float>(), ids.numel(),
                    (int)grad_table.size(1), grad_table.size(0), is_bf16(g), stream());
}

void embedding_bwd_sorted_(const Tensor& sorted_ids, const Tensor& perm, const Tensor& g, Tensor& grad_table) {
  CHECK_CUDA_CONTIG(sorted_ids);
  CHECK_CUDA_CONTIG(perm);
  CHECK_CUDA_CONTIG(g);
  CHECK_CUDA_CONTIG(grad_table);
  TORCH_CHECK(grad_table.scalar_type() == at::kFloat, "embedding_bwd_sorted_: fp32 accumulation buffer expected");
  TORCH_CHECK(sorted_ids.scalar_type() == at::kLong && perm.scalar_type() == at::kLong && perm.numel() == sorted_ids.numel(),
              "embedding_bwd_sorted_: int64 ids and permutation of the same length");
  const c10::cuda::CUDAGuard guard(g.device());
  count();
  ab::embedding_bwd_sorted((const long long*)sorted_ids.data_ptr<int64_t>(), (const long long*)perm.data_ptr<int64_t>(),
                           g.data_ptr(), grad_table.data_ptr<float>(), sorted_ids.numel(), (int)grad_table.size(1),
                           grad_table.size(0), is_bf16(g), stream());
}

// logits [rows, V] (unit column stride).  Writes the gradient over `logits` when in_place_grad (scaled by grad_scale[0]).
std::tuple<Tensor, Tensor> ce_rows(Tensor& logits, const Tensor& targets, double smoothing, int64_t ignore_index,
                                   const c10::optional<Tensor>& grad_scale, bool in_place_grad) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "ce_rows: logits must be [rows, V]");
  CHECK_CUDA_CONTIG(targets);
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.numel() == logits.size(0), "ce_rows: targets int64 [rows]");
  TORCH_CHECK(!in_place_grad || grad_scale.has_value(), "ce_rows: grad_scale required for the gradient");
  const c10::cuda::CUDAGuard guard(logits.device());
  const long long rows = logits.size(0);
  Tensor loss = at::empty({rows}, logits.options().dtype(at::kFloat));
  Tensor logprob = at::empty({rows}, loss.options());
  count();
  ab::ce_rows(logits.data_ptr(), in_place_grad ? logits.data_ptr() : nullptr, (const long long*)targets.data_ptr<int64_t>(),
              loss.data_ptr<float>(), logprob.data_ptr<float>(),
              grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, rows, (int)logits.size(1),
              logits.stride(0), (float)smoothing, ignore_index, is_bf16(logits), stream());
  return {loss, logprob};
}

void logprob_bwd_(Tensor& logits, const Tensor& targets, const Tensor& logprob, const Tensor& g_rows) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "logprob_bwd_: logits must be [rows, V]");
  const c10::cuda::CUDAGuard guard(logits.device());
  count();
  ab::logprob_bwd(logits.data_ptr(), logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(),
                  logprob.data_ptr<float>(), g_rows.data_ptr<float>(), logits.size(0), (int)logits.size(1),
                  logits.stride(0), is_bf16(logits), stream());
}

void sumsq_(const Tensor& x, Tensor& out) {
  CHECK_CUDA_CONTIG(x);
  const c10::cuda::CUDAGuard guard(x.device());
  count();
  ab::sumsq_accum(x.data_ptr(), x.numel(), out.data_ptr<float>(), is_bf16(x), stream());
}

void clip_coef_(const Tensor& sumsq, double max_norm, double pre_scale, Tensor& coef, Tensor& norm) {
  const c10::cuda::CUDAGuard guard(sumsq.device());
  count();
  ab::clip_coef(sumsq.data_ptr<float>(), (float)max_norm, (float)pre_scale, coef.data_ptr<float>(),
                norm.data_ptr<float>(), stream());
}

void adamw_(Tensor& p, const c10::optional<Tensor>& master, Tensor& g, Tensor& m, Tensor& v, double lr, double b1,
            double b2, double eps, double wd, int64_t step, const c10::optional<Tensor>& gscale, bool zero_grad) {
  CHECK_CUDA_CONTIG(p);
  CHECK_CUDA_CONTIG(g);
  TORCH_CHECK(g.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat,
              "adamw_: gradient and moments are fp32");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "adamw_: size mismatch");
  const c10::cuda::CUDAGuard guard(p.device());
  count();
  ab::adamw_step(p.data_ptr(), master.has_value() ? master->data_ptr<float>() : nullptr, g.data_ptr<float>(),
                 m.data_ptr<float>(), v.data_ptr<float>(), p.numel(), (float)lr, (float)b1, (float)b2, (float)eps,
                 (float)wd, (int)step, gscale.has_value() ? gscale->data_ptr<float>() : nullptr, zero_grad, is_bf16(p),
                 stream());
}

void axpy_f32_(Tensor& dst, const Tensor& src, double alpha) {
  CHECK_CUDA_CONTIG(dst);
  CHECK_CUDA_CONTIG(src);
  TORCH_CHECK(dst.scalar_type() == at::kFloat && dst.numel() == src.numel(), "axpy_f32_: fp32 destination, equal sizes");
  const c10::cuda::CUDAGuard guard(dst.device());
  count();
  ab::axpy_f32(dst.data_ptr<float>(), src.data_ptr(), dst.numel(), (float)alpha, is_bf16(src), stream());
}

Tensor& status_tensor(const at::Device& dev) {
  static std::map<int, Tensor> per_device;
  auto it = per_device.find(dev.index());
  if (it == per_device.end())
    it = per_device.emplace(dev.index(), at::zeros({4}, at::TensorOptions().device(dev).dtype(at::kInt))).first;
  return it->second;
}

Tensor kernel_status(const Tensor& like) { return status_tensor(like.device()); }

// D[M,N] (+)= op(A) x op(B).  A is [M,K] (a_kmajor) or [K,M]; B is [N,K] (b_kmajor) or [K,N]; all 2-D, unit column stride.
Tensor gemm(const Tensor& A, const Tensor& B, const c10::optional<Tensor>& D_in, bool a_kmajor, bool b_kmajor,
            bool out_f32, bool accumulate) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && A.dim() == 2 && B.dim() == 2 && A.stride(1) == 1 && B.stride(1) == 1,
              "gemm: operands must be 2-D CUDA tensors with unit column stride");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: bf16 operands");
  const c10::cuda::CUDAGuard guard(A.device());
  const int M = (int)(a_kmajor ? A.size(0) : A.size(1)), K = (int)(a_kmajor ? A.size(1) : A.size(0));
  const int N = (int)(b_kmajor ? B.size(0) : B.size(1)), Kb = (int)(b_kmajor ? B.size(1) : B.size(0));
  TORCH_CHECK(K == Kb, "gemm: inner dimensions differ (", K, " vs ", Kb, ")");
  Tensor D;
  if (D_in.has_value()) {
    D = *D_in;
    TORCH_CHECK(D.dim() == 2 && D.size(0) == M && D.size(1) == N && D.stride(1) == 1, "gemm: bad output shape");
    TORCH_CHECK(D.scalar_type() == (out_f32 ? at::kFloat : at::kBFloat16), "gemm: output dtype mismatch");
  } else {
    TORCH_CHECK(!accumulate, "gemm: accumulate needs an output tensor");
    D = at::empty({M, N}, A.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  }
  if (a_kmajor && b_kmajor && !out_f32 && !accumulate && M <= 256 && N >= 128 && K >= 128) {
    // decode-sized batch: stream the weight through all SMs (weight = MMA M operand, K split over a cluster)
    count();
    const int rcs = ab::gemm_skinny(A.data_ptr(), B.data_ptr(), D.data_ptr(), M, N, K, A.stride(0), B.stride(0), D.stride(0),
                                    status_tensor(A.device()).data_ptr<int>(), stream());
    TORCH_CHECK(rcs == 0, "gemm_skinny launch failed with code ", rcs);
    return D;
  }
  count();
  const int rc = ab::gemm_bf16(A.data_ptr(), B.data_ptr(), D.data_ptr(), M, N, K, A.stride(0), B.stride(0), D.stride(0),
                               a_kmajor, b_kmajor, out_f32, accumulate, status_tensor(A.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_bf16 launch failed with code ", rc,
              " (-1: operand not 16-byte aligned / stride not a multiple of 8, -2: tensor map, -4/-5: launch)");
  return D;
}

// k_new/v_new [T, Hkv, D] contiguous bf16; k_buf/v_buf [n_slots, Hkv, D]; loc int32 [T]
void kv_append_(const Tensor& k_new, const Tensor& v_new, Tensor& k_buf, Tensor& v_buf, const Tensor& loc) {
  CHECK_CUDA_CONTIG(k_new);
  CHECK_CUDA_CONTIG(v_new);
  CHECK_CUDA_CONTIG(k_buf);
  CHECK_CUDA_CONTIG(v_buf);
  CHECK_CUDA_CONTIG(loc);
  TORCH_CHECK(k_new.scalar_type() == at::kBFloat16 && k_buf.scalar_type() == at::kBFloat16, "kv_append_: bf16 only");
  TORCH_CHECK(loc.scalar_type() == at::kInt && loc.numel() == k_new.size(0), "kv_append_: loc must be int32 [tokens]");
  const int row = (int)(k_buf.size(1) * k_buf.size(2));
  TORCH_CHECK(row % 8 == 0 && k_new.numel() == k_new.size(0) * row && v_new.numel() == k_new.numel(), "kv_append_: row mismatch");
  const c10::cuda::CUDAGuard guard(k_buf.device());
  count();
  ab::kv_append(k_new.data_ptr(), v_new.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), loc.data_ptr<int>(), k_new.size(0),
                row, k_buf.size(0), stream());
}

int64_t paged_decode_splits(int64_t batch, int64_t n_kv_heads, int64_t max_len, int64_t max_splits) {
  return ab::paged_decode_splits((int)batch, (int)n_kv_heads, max_len, (int)max_splits);
}

// q [B, Hq, D]; scratch: o_part [>=B, Hq, max_splits, D] f32, ml_part [>=B, Hq, max_splits, 2] f32, counters int32 [>=B*Hkv] (zero)
void paged_decode_impl(const Tensor& q, const Tensor& k_buf, const Tensor& v_buf, const Tensor& req_to_token,
                       const Tensor& req_pool_indices, const Tensor& seq_lens, double scale, int64_t splits, Tensor& o_part,
                       Tensor& ml_part, Tensor& counters, Tensor& out, const Tensor* k_new, const Tensor* v_new) {
  CHECK_CUDA_CONTIG(q);
  CHECK_CUDA_CONTIG(k_buf);
  CHECK_CUDA_CONTIG(v_buf);
  CHECK_CUDA_CONTIG(req_to_token);
  CHECK_CUDA_CONTIG(out);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k_buf.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "paged_decode_: bf16 only");
  TORCH_CHECK(req_to_token.scalar_type() == at::kInt && req_pool_indices.scalar_type() == at::kInt && seq_lens.scalar_type() == at::kLong,
              "paged_decode_: req_to_token/req_pool_indices int32, seq_lens int64");
  const int B = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)k_buf.size(1);
  const int max_splits = (int)o_part.size(2);
  TORCH_CHECK(o_part.scalar_type() == at::kFloat && o_part.size(0) >= B && o_part.size(1) == Hq && o_part.size(3) == D, "paged_decode_: bad o_part scratch");
  TORCH_CHECK(ml_part.scalar_type() == at::kFloat && ml_part.size(0) >= B && ml_part.size(2) == max_splits, "paged_decode_: bad ml_part scratch");
  TORCH_CHECK(counters.scalar_type() == at::kInt && counters.numel() >= (int64_t)B * Hkv, "paged_decode_: bad counters scratch");
  if (k_new != nullptr) {
    TORCH_CHECK(k_new->is_cuda() && k_new->is_contiguous() && v_new->is_cuda() && v_new->is_contiguous() &&
                k_new->scalar_type() == at::kBFloat16 && v_new->scalar_type() == at::kBFloat16 && k_new->dim() == 3 &&
                k_new->size(0) == B && k_new->size(1) == Hkv && k_new->size(2) == D && v_new->sizes() == k_new->sizes(),
                "paged_decode_append_: k_new / v_new must be contiguous bf16 [batch, kv_heads, head_dim]");
  }
  const c10::cuda::CUDAGuard guard(q.device());
  count();
  const int rc = ab::paged_decode(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), req_to_token.data_ptr<int>(),
                                  req_pool_indices.data_ptr<int>(), (const long long*)seq_lens.data_ptr<int64_t>(),
                                  o_part.data_ptr<float>(), ml_part.data_ptr<float>(), counters.data_ptr<int>(), out.data_ptr(),
                                  B, Hq, Hkv, D, (int)req_to_token.size(1), k_buf.size(0), (float)scale, (int)splits, max_splits,
                                  (int)req_to_token.size(0), stream(), k_new ? k_new->data_ptr() : nullptr,
                                  v_new ? v_new->data_ptr() : nullptr);
  TORCH_CHECK(rc == 0, "paged_decode launch failed with code ", rc, " (-1: more than 8 query heads per kv head, -2: splits, -3: head_dim not in {32,64,128,256})");
}

void paged_decode_(const Tensor& q, const Tensor& k_buf, const Tensor& v_buf, const Tensor& req_to_token,
                   const Tensor& req_pool_indices, const Tensor& seq_lens, double scale, int64_t splits, Tensor& o_part,
                   Tensor& ml_part, Tensor& counters, Tensor& out) {
  paged_decode_impl(q, k_buf, v_buf, req_to_token, req_pool_indices, seq_lens, scale, splits, o_part, ml_part, counters, out,
                    nullptr, nullptr);
}

// Decode attention with the step's K / V append fused in: k_new / v_new [batch, Hkv, D] are read for the last position
// and stored into the pool slot the table names for it (one launch instead of kv_append_ + paged_decode_).
void paged_decode_append_(const Tensor& q, const Tensor& k_new, const Tensor& v_new, Tensor& k_buf, Tensor& v_buf,
                          const Tensor& req_to_token, const Tensor& req_pool_indices, const Tensor& seq_lens, double scale,
                          int64_t splits, Tensor& o_part, Tensor& ml_part, Tensor& counters, Tensor& out) {
  paged_decode_impl(q, k_buf, v_buf, req_to_token, req_pool_indices, seq_lens, scale, splits, o_part, ml_part, counters, out,
                    &k_new, &v_new);
}

// q [Tq, Hq, D], k / v [Tk, Hkv, D] packed along tokens (a dense [B,S,H,D] batch is the same memory).
std::tuple<Tensor, Tensor> flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& cu_q,
                                     const c10::optional<Tensor>& cu_k, int64_t batch, int64_t sq, int64_t sk,
                                     int64_t max_q, bool causal, double scale) {
  auto ok = [](const Tensor& t) {
    return t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kBFloat16 && t.stride(2) == 1 && t.stride(1) == t.size(2) &&
           t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(ok(q) && ok(k) && ok(v), "flash_fwd: q/k/v must be bf16 [tokens, heads, D] with adjacent heads, 16-byte aligned");
  TORCH_CHECK(k.size(0) == v.size(0) && k.size(1) == v.size(1) && q.size(2) == k.size(2) && k.size(2) == v.size(2), "flash_fwd: shape mismatch");
  const int D = (int)q.size(2);
  TORCH_CHECK(D == 64 || D == 128, "flash_fwd: head_dim must be 64 or 128");
  const int* cq = nullptr;
  const int* ck = nullptr;
  if (cu_q.has_value()) {
    TORCH_CHECK(cu_q->is_cuda() && cu_q->scalar_type() == at::kInt && cu_q->numel() == batch + 1, "flash_fwd: cu_q int32 [batch+1]");
    cq = cu_q->data_ptr<int>();
  } else {
    TORCH_CHECK(batch * sq == q.size(0), "flash_fwd: batch * sq must equal the number of query tokens");
  }
  if (cu_k.has_value()) {
    TORCH_CHECK(cu_k->is_cuda() && cu_k->scalar_type() == at::kInt && cu_k->numel() == batch + 1, "flash_fwd: cu_k int32 [batch+1]");
    ck = cu_k->data_ptr<int>();
  } else {
    TORCH_CHECK(batch * sk == k.size(0), "flash_fwd: batch * sk must equal the number of key tokens");
  }
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({q.size(0), q.size(1), q.size(2)}, q.options());
  Tensor lse = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  count();
  const int rc = ab::flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), cq, ck,
                               (int)batch, (int)sq, (int)sk, (int)max_q, q.size(0), k.size(0), (int)q.size(1), (int)k.size(1), D,
                               q.stride(0), k.stride(0), v.stride(0), out.stride(0), (float)scale, causal,
                               status_tensor(q.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "flash_fwd launch failed with code ", rc);
  return {out, lse};
}

// Prefill over the paged KV pool without gathering: q [Tq, Hq, D] packed queries (cu_q), k_pool / v_pool [n_slots, Hkv, D],
// kv_lens through cu_k (differences), slot table [rows, max_ctx] + req_pool_indices [batch]; causal is lower-right aligned.
Tensor flash_fwd_paged(const Tensor& q, const Tensor& k_pool, const Tensor& v_pool, const Tensor& cu_q, const Tensor& cu_k,
                       const Tensor& table, const Tensor& rows, int64_t page, int64_t max_q, bool causal, double scale) {
  auto ok = [](const Tensor& t) {
    return t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kBFloat16 && t.stride(2) == 1 && t.stride(1) == t.size(2) &&
           t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(ok(q) && ok(k_pool) && ok(v_pool), "flash_fwd_paged: bf16 [tokens, heads, D] tensors with adjacent heads, 16-byte aligned");
  TORCH_CHECK(k_pool.sizes() == v_pool.sizes() && q.size(2) == k_pool.size(2), "flash_fwd_paged: shape mismatch");
  const int D = (int)q.size(2);
  TORCH_CHECK(D == 64 || D == 128, "flash_fwd_paged: head_dim must be 64 or 128");
  TORCH_CHECK(page == 8 || page == 16 || page == 32 || page == 64, "flash_fwd_paged: page size must be 8, 16, 32 or 64");
  const int64_t batch = cu_q.numel() - 1;
  TORCH_CHECK(cu_q.is_cuda() && cu_q.scalar_type() == at::kInt && cu_k.is_cuda() && cu_k.scalar_type() == at::kInt &&
              cu_k.numel() == batch + 1 && batch >= 1, "flash_fwd_paged: cu_q / cu_k int32 [batch+1]");
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kInt && table.dim() == 2 && table.is_contiguous() &&
              rows.is_cuda() && rows.scalar_type() == at::kInt && rows.numel() >= batch, "flash_fwd_paged: table int32 [rows, ctx], rows int32 [batch]");
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({q.size(0), q.size(1), q.size(2)}, q.options());
  ab::PagedKv pg;
  pg.table = table.data_ptr<int>(), pg.rows = rows.data_ptr<int>(), pg.stride = table.size(1), pg.page = (int)page;
  count();
  const int rc = ab::flash_fwd(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), nullptr, cu_q.data_ptr<int>(),
                               cu_k.data_ptr<int>(), (int)batch, 0, 0, (int)max_q, q.size(0), k_pool.size(0), (int)q.size(1),
                               (int)k_pool.size(1), D, q.stride(0), k_pool.stride(0), v_pool.stride(0), out.stride(0), (float)scale,
                               causal, status_tensor(q.device()).data_ptr<int>(), stream(), nullptr, &pg);
  TORCH_CHECK(rc == 0, "flash_fwd_paged launch failed with code ", rc);
  return out;
}

std::tuple<Tensor, Tensor, Tensor> flash_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                                             const Tensor& dout, const Tensor& lse, const c10::optional<Tensor>& cu_q,
                                             const c10::optional<Tensor>& cu_k, int64_t batch, int64_t sq, int64_t sk,
                                             int64_t max_q, int64_t max_k, bool causal, double scale) {
  auto ok = [](const Tensor& t) {
    return t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kBFloat16 && t.stride(2) == 1 && t.stride(1) == t.size(2) &&
           t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(ok(q) && ok(k) && ok(v) && ok(out) && ok(dout), "flash_bwd: tensors must be bf16 [tokens, heads, D] with adjacent heads");
  TORCH_CHECK(lse.is_cuda() && lse.is_contiguous() && lse.scalar_type() == at::kFloat && lse.numel() == q.size(0) * q.size(1), "flash_bwd: lse [Hq, tokens] fp32");
  const int D = (int)q.size(2);
  TORCH_CHECK(D == 64 || D == 128, "flash_bwd: head_dim must be 64 or 128");
  const int* cq = cu_q.has_value() ? cu_q->data_ptr<int>() : nullptr;
  const int* ck = cu_k.has_value() ? cu_k->data_ptr<int>() : nullptr;
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor dq = at::empty({q.size(0), q.size(1), q.size(2)}, q.options());
  Tensor dk = at::empty({k.size(0), k.size(1), k.size(2)}, k.options());
  Tensor dv = at::empty({k.size(0), k.size(1), k.size(2)}, k.options());
  Tensor delta = at::empty({2, q.size(1), q.size(0)}, q.options().dtype(at::kFloat));  // row dots | lse in log2 units
  count(3);
  const int rc = ab::flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(),
                               delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cq, ck, (int)batch, (int)sq,
                               (int)sk, (int)max_q, (int)max_k, q.size(0), k.size(0), (int)q.size(1), (int)k.size(1), D,
                               q.stride(0), k.stride(0), v.stride(0), out.stride(0), dout.stride(0), dq.stride(0), dk.stride(0),
                               (float)scale, causal, status_tensor(q.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "flash_bwd launch failed with code ", rc);
  return {dq, dk, dv};
}

// ---- context-parallel flash attention (zig-zag sequence sharding, see CpAttn in launchers.h).
// q / out are the rank's 2 * chunk rows per batch entry, k_full / v_full the gathered [batch * S, Hkv, D] keys.
ab::CpAttn cp_params(int64_t batch, int64_t chunk, int64_t world, int64_t rank, const std::vector<int64_t>& flag_ptrs,
                     int64_t unit, int64_t max_units, int64_t epoch, double timeout_s) {
  TORCH_CHECK(world >= 2 && world <= 8 && rank >= 0 && rank < world, "context parallel: world in 2..8, rank in range");
  TORCH_CHECK(chunk > 0 && chunk % 128 == 0, "context parallel: chunk must be a positive multiple of 128");
  ab::CpAttn cp;
  cp.world = (int)world, cp.rank = (int)rank, cp.chunk = (int)chunk, cp.batch = (int)batch;
  cp.k_vis = (int)((2 * world - rank) * chunk);
  cp.unit = (int)unit, cp.max_units = (int)max_units, cp.epoch = (int)epoch;
  cp.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  TORCH_CHECK(flag_ptrs.empty() || (int64_t)flag_ptrs.size() == world, "context parallel: one flag pointer per rank");
  for (size_t i = 0; i < flag_ptrs.size(); ++i) cp.flags[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  return cp;
}

std::tuple<Tensor, Tensor> cp_flash_fwd(const Tensor& q, const Tensor& k_full, const Tensor& v_full, int64_t batch,
                                        int64_t chunk, int64_t world, int64_t rank, double scale,
                                        std::vector<int64_t> kv_src_ptrs, std::vector<int64_t> flag_ptrs, int64_t unit,
                                        int64_t max_units, int64_t epoch, int64_t n_copy_ctas,
                                        const c10::optional<Tensor>& chunk_state, double timeout_s) {
  auto ok = [](const Tensor& t) {
    return t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kBFloat16 && t.is_contiguous() &&
           (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(ok(q) && ok(k_full) && ok(v_full), "cp_flash_fwd: contiguous bf16 [tokens, heads, D] tensors");
  const int64_t S = 2 * world * chunk;
  TORCH_CHECK(q.size(0) == batch * 2 * chunk && k_full.size(0) == batch * S && v_full.sizes() == k_full.sizes(), "cp_flash_fwd: shapes");
  const int D = (int)q.size(2);
  ab::CpAttn cp = cp_params(batch, chunk, world, rank, flag_ptrs, unit, max_units, epoch, timeout_s);
  if (!kv_src_ptrs.empty()) {
    TORCH_CHECK((int64_t)kv_src_ptrs.size() == world && (int64_t)flag_ptrs.size() == world, "cp_flash_fwd: one source / flag pointer per rank");
    TORCH_CHECK(chunk_state.has_value() && chunk_state->is_cuda() && chunk_state->scalar_type() == at::kInt && chunk_state->numel() >= 16, "cp_flash_fwd: chunk_state int32 [16]");
    for (int64_t i = 0; i < world; ++i) cp.kv_src[i] = reinterpret_cast<const void*>(kv_src_ptrs[i]);
    cp.k_full = k_full.data_ptr(), cp.v_full = v_full.data_ptr();
    cp.chunk_flags = chunk_state->data_ptr<int>(), cp.chunk_counter = chunk_state->data_ptr<int>() + 8;
    cp.n_copy_ctas = (int)n_copy_ctas;
  }
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty_like(q);
  Tensor lse = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  count();
  const int rc = ab::flash_fwd(q.data_ptr(), k_full.data_ptr(), v_full.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), nullptr,
                               nullptr, (int)batch, (int)(2 * chunk), (int)S, (int)(2 * chunk), q.size(0), k_full.size(0),
                               (int)q.size(1), (int)k_full.size(1), D, q.stride(0), k_full.stride(0), v_full.stride(0),
                               out.stride(0), (float)scale, true, status_tensor(q.device()).data_ptr<int>(), stream(), &cp);
  TORCH_CHECK(rc == 0, "cp_flash_fwd launch failed with code ", rc);
  return {out, lse};
}

// Returns dq and, when no staging pointers are given, this rank's partial dk / dv over the gathered keys (zero where it
// sees nothing); with staging pointers the partials go to their owners and two empty tensors come back.
std::tuple<Tensor, Tensor, Tensor> cp_flash_bwd(const Tensor& q, const Tensor& k_full, const Tensor& v_full, const Tensor& out,
                                                const Tensor& dout, const Tensor& lse, int64_t batch, int64_t chunk,
                                                int64_t world, int64_t rank, double scale, std::vector<int64_t> stage_ptrs,
                                                std::vector<int64_t> flag_ptrs, int64_t unit, int64_t max_units, int64_t epoch,
                                                const c10::optional<Tensor>& tile_counter, double timeout_s) {
  auto ok = [](const Tensor& t) {
    return t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kBFloat16 && t.is_contiguous() &&
           (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(ok(q) && ok(k_full) && ok(v_full) && ok(out) && ok(dout), "cp_flash_bwd: contiguous bf16 [tokens, heads, D] tensors");
  const int64_t S = 2 * world * chunk;
  TORCH_CHECK(q.size(0) == batch * 2 * chunk && k_full.size(0) == batch * S && v_full.sizes() == k_full.sizes(), "cp_flash_bwd: shapes");
  const int D = (int)q.size(2);
  ab::CpAttn cp = cp_params(batch, chunk, world, rank, flag_ptrs, unit, max_units, epoch, timeout_s);
  const bool scatter = !stage_ptrs.empty();
  if (scatter) {
    TORCH_CHECK((int64_t)stage_ptrs.size() == world && (int64_t)flag_ptrs.size() == world, "cp_flash_bwd: one staging / flag pointer per rank");
    TORCH_CHECK(tile_counter.has_value() && tile_counter->is_cuda() && tile_counter->scalar_type() == at::kInt && tile_counter->numel() >= 8, "cp_flash_bwd: tile_counter int32 [8]");
    for (int64_t i = 0; i < world; ++i) cp.stage[i] = reinterpret_cast<void*>(stage_ptrs[i]);
    cp.tile_counter = tile_counter->data_ptr<int>();
  }
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor dq = at::empty_like(q);
  Tensor dk = scatter ? at::empty({0}, q.options()) : at::zeros_like(k_full);
  Tensor dv = scatter ? at::empty({0}, q.options()) : at::zeros_like(v_full);
  Tensor delta = at::empty({2, q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  count(3);
  const int rc = ab::flash_bwd(q.data_ptr(), k_full.data_ptr(), v_full.data_ptr(), out.data_ptr(), dout.data_ptr(),
                               lse.data_ptr<float>(), delta.data_ptr<float>(), dq.data_ptr(), scatter ? nullptr : dk.data_ptr(),
                               scatter ? nullptr : dv.data_ptr(), nullptr, nullptr, (int)batch, (int)(2 * chunk), (int)S,
                               (int)(2 * chunk), cp.k_vis, q.size(0), k_full.size(0), (int)q.size(1), (int)k_full.size(1), D,
                               q.stride(0), k_full.stride(0), v_full.stride(0), out.stride(0), dout.stride(0), dq.stride(0),
                               k_full.stride(0), (float)scale, true, status_tensor(q.device()).data_ptr<int>(), stream(), &cp);
  TORCH_CHECK(rc == 0, "cp_flash_bwd launch failed with code ", rc);
  return {dq, dk, dv};
}

void cp_dkv_reduce(Tensor dk_local, Tensor dv_local, int64_t batch, int64_t chunk, int64_t world, int64_t rank,
                   std::vector<int64_t> stage_ptrs, std::vector<int64_t> flag_ptrs, int64_t unit, int64_t max_units,
                   int64_t epoch, double timeout_s) {
  TORCH_CHECK(dk_local.is_cuda() && dk_local.is_contiguous() && dk_local.scalar_type() == at::kBFloat16 && dk_local.dim() == 3 &&
                  dv_local.is_contiguous() && dv_local.sizes() == dk_local.sizes() && dv_local.scalar_type() == at::kBFloat16,
              "cp_dkv_reduce: contiguous bf16 [batch * 2 * chunk, Hkv, D] outputs");
  TORCH_CHECK(dk_local.size(0) == batch * 2 * chunk && (int64_t)stage_ptrs.size() == world && (int64_t)flag_ptrs.size() == world, "cp_dkv_reduce: shapes");
  ab::CpAttn cp = cp_params(batch, chunk, world, rank, flag_ptrs, unit, max_units, epoch, timeout_s);
  for (int64_t i = 0; i < world; ++i) cp.stage[i] = reinterpret_cast<void*>(stage_ptrs[i]);
  const c10::cuda::CUDAGuard guard(dk_local.device());
  count();
  const int rc = ab::cp_dkv_reduce(dk_local.data_ptr(), dv_local.data_ptr(), (int)batch, (int)(dk_local.size(1) * dk_local.size(2)),
                                   cp, status_tensor(dk_local.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "cp_dkv_reduce launch failed with code ", rc);
}

// ---- fused FSDP over peer memory.  Pointer lists are raw device addresses of the same symmetric buffer on each rank.
ab::CommPeers peers_from(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && ptrs.size() <= 8, "peer pointer list must have 1..8 entries");
  ab::CommPeers p{};
  for (size_t i = 0; i < ptrs.size(); ++i) p.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return p;
}

void fsdp_reduce_scatter_(std::vector<int64_t> grad_ptrs, int64_t mc_ptr, std::vector<int64_t> flag_ptrs, int64_t rank,
                          int64_t shard_off, Tensor& out, Tensor& sumsq, int64_t unit, int64_t max_units, int64_t epoch,
                          double timeout_s, int64_t max_ctas) {
  CHECK_CUDA_CONTIG(out);
  TORCH_CHECK(out.scalar_type() == at::kFloat && sumsq.scalar_type() == at::kFloat, "fsdp_reduce_scatter_: fp32 buffers");
  TORCH_CHECK(grad_ptrs.size() == flag_ptrs.size(), "fsdp_reduce_scatter_: pointer lists differ in length");
  const c10::cuda::CUDAGuard guard(out.device());
  count();
  const int rc = ab::fsdp_reduce_scatter(peers_from(grad_ptrs), reinterpret_cast<const float*>(mc_ptr), peers_from(flag_ptrs),
                                         (int)grad_ptrs.size(), (int)rank, shard_off, out.numel(), out.data_ptr<float>(),
                                         sumsq.data_ptr<float>(), (int)unit, (int)max_units, (int)epoch,
                                         (unsigned long long)(timeout_s * 1e9), status_tensor(out.device()).data_ptr<int>(),
                                         (int)max_ctas, stream());
  TORCH_CHECK(rc == 0, "fsdp_reduce_scatter launch failed with code ", rc);
}

void fsdp_adamw_allgather_(std::vector<int64_t> param_ptrs, int64_t mc_ptr, std::vector<int64_t> flag_ptrs, int64_t rank,
                           int64_t shard_off, const c10::optional<Tensor>& master, const Tensor& g, Tensor& m, Tensor& v,
                           double lr, double b1, double b2, double eps, double wd, int64_t step,
                           const c10::optional<Tensor>& gscale, int64_t unit, int64_t max_units, int64_t epoch,
                           Tensor& block_counter, int64_t max_ctas) {
  CHECK_CUDA_CONTIG(g);
  TORCH_CHECK(g.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat,
              "fsdp_adamw_allgather_: gradient and moments are fp32");
  TORCH_CHECK(m.numel() == g.numel() && v.numel() == g.numel(), "fsdp_adamw_allgather_: size mismatch");
  TORCH_CHECK(block_counter.scalar_type() == at::kInt && block_counter.numel() >= 1, "fsdp_adamw_allgather_: counter");
  const c10::cuda::CUDAGuard guard(g.device());
  count();
  const int rc = ab::fsdp_adamw_allgather(peers_from(param_ptrs), reinterpret_cast<void*>(mc_ptr), peers_from(flag_ptrs),
                                          (int)param_ptrs.size(), (int)rank, shard_off, g.numel(),
                                          master.has_value() ? master->data_ptr<float>() : nullptr, g.data_ptr<float>(),
                                          m.data_ptr<float>(), v.data_ptr<float>(), (float)lr, (float)b1, (float)b2,
                                          (float)eps, (float)wd, (int)step,
                                          gscale.has_value() ? gscale->data_ptr<float>() : nullptr, (int)unit,
                                          (int)max_units, (int)epoch, block_counter.data_ptr<int>(), (int)max_ctas, stream());
  TORCH_CHECK(rc == 0, "fsdp_adamw_allgather launch failed with code ", rc);
}

void comm_wait_flags_(const Tensor& local_flags, int64_t kind, int64_t world, int64_t skip_rank, int64_t unit,
                      int64_t max_units, int64_t epoch, double timeout_s) {
  TORCH_CHECK(local_flags.is_cuda() && local_flags.scalar_type() == at::kInt, "comm_wait_flags_: int32 CUDA flags");
  const c10::cuda::CUDAGuard guard(local_flags.device());
  count();
  const int rc = ab::comm_wait_flags(local_flags.data_ptr<int>(), (int)kind, (int)world, (int)skip_rank, (int)unit,
                                     (int)max_units, (int)epoch, (unsigned long long)(timeout_s * 1e9),
                                     status_tensor(local_flags.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "comm_wait_flags launch failed with code ", rc);
}

// ---- tensor-parallel fused GEMMs.  Pointer lists: the same symmetric buffer on every rank.
void fill_ptrs(void* (&dst)[8], const std::vector<int64_t>& src) {
  TORCH_CHECK(src.size() >= 1 && src.size() <= 8, "peer pointer list must have 1..8 entries");
  for (size_t i = 0; i < 8; ++i) dst[i] = i < src.size() ? reinterpret_cast<void*>(src[i]) : nullptr;
}

void tp_gemm_allgather_(std::vector<int64_t> xfull_ptrs, const Tensor& W, bool w_kmajor, Tensor& Y, std::vector<int64_t> flag_ptrs,
                        Tensor& chunk_flags, Tensor& chunk_counter, int64_t rank, int64_t unit, int64_t max_units,
                        int64_t epoch, double timeout_s, int64_t n_copy_ctas) {
  CHECK_CUDA_CONTIG(W);
  CHECK_CUDA_CONTIG(Y);
  TORCH_CHECK(W.scalar_type() == at::kBFloat16 && Y.scalar_type() == at::kBFloat16 && W.dim() == 2 && Y.dim() == 2, "tp_gemm_allgather_: bf16 2-D");
  TORCH_CHECK(chunk_flags.scalar_type() == at::kInt && chunk_flags.numel() >= 8 && chunk_counter.scalar_type() == at::kInt && chunk_counter.numel() >= 8, "tp_gemm_allgather_: int32[8] flags / counters");
  const int64_t N = w_kmajor ? W.size(0) : W.size(1), K = w_kmajor ? W.size(1) : W.size(0);
  TORCH_CHECK(Y.size(1) == N, "tp_gemm_allgather_: output columns must match the weight");
  ab::TpGemmParams p{};
  p.world = (int)xfull_ptrs.size(); p.rank = (int)rank; p.unit = (int)unit; p.max_units = (int)max_units; p.epoch = (int)epoch;
  p.n_copy_ctas = (int)n_copy_ctas; p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  fill_ptrs(p.flags, flag_ptrs); fill_ptrs(p.x_full, xfull_ptrs);
  p.chunk_flags = chunk_flags.data_ptr<int>(); p.chunk_counter = chunk_counter.data_ptr<int>();
  const c10::cuda::CUDAGuard guard(W.device());
  count();
  const int rc = ab::gemm_allgather(W.data_ptr(), w_kmajor, Y.data_ptr(), (int)Y.size(0), (int)N, (int)K, Y.stride(0), p,
                                    status_tensor(W.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_allgather launch failed with code ", rc, " (-2: M must be a multiple of world*128, N of 32, K of 8)");
}

void tp_gemm_reducescatter_(const Tensor& X, const Tensor& W, bool w_kmajor, std::vector<int64_t> stage_ptrs, Tensor& out,
                            std::vector<int64_t> flag_ptrs, Tensor& tile_counter, int64_t rank, int64_t unit,
                            int64_t max_units, int64_t epoch, double timeout_s, bool fuse_reduce) {
  CHECK_CUDA_CONTIG(X);
  CHECK_CUDA_CONTIG(W);
  CHECK_CUDA_CONTIG(out);
  TORCH_CHECK(X.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16, "tp_gemm_reducescatter_: bf16");
  const int64_t N = w_kmajor ? W.size(0) : W.size(1), K = w_kmajor ? W.size(1) : W.size(0);
  TORCH_CHECK(X.dim() == 2 && W.dim() == 2 && X.size(1) == K, "tp_gemm_reducescatter_: inner dimensions differ");
  TORCH_CHECK(tile_counter.scalar_type() == at::kInt && tile_counter.numel() >= 8, "tp_gemm_reducescatter_: int32[8] counter");
  ab::TpGemmParams p{};
  p.world = (int)stage_ptrs.size(); p.rank = (int)rank; p.unit = (int)unit; p.max_units = (int)max_units; p.epoch = (int)epoch;
  p.fuse_reduce = fuse_reduce ? 1 : 0; p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  TORCH_CHECK(out.size(0) * p.world == X.size(0) && out.size(1) == N, "tp_gemm_reducescatter_: output must be [M/world, N]");
  fill_ptrs(p.flags, flag_ptrs); fill_ptrs(p.stage, stage_ptrs);
  p.rs_out = out.data_ptr(); p.tile_counter = tile_counter.data_ptr<int>();
  const c10::cuda::CUDAGuard guard(X.device());
  count();
  const int rc = ab::gemm_reducescatter(X.data_ptr(), W.data_ptr(), w_kmajor, (int)X.size(0), (int)N, (int)K, p,
                                        status_tensor(X.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_reducescatter launch failed with code ", rc, " (-2: M must be a multiple of world*128, N of 32, K of 8)");
}

// The pair-tile engine (gemm_comm2.cu): the transfer runs as bulk copies issued by one extra warp of every GEMM CTA.
void tp2_gemm_allgather_(std::vector<int64_t> xfull_ptrs, const Tensor& W, bool w_kmajor, Tensor& Y, std::vector<int64_t> flag_ptrs,
                         Tensor& chunk_flags, Tensor& chunk_counter, int64_t rank, int64_t unit, int64_t max_units,
                         int64_t epoch, double timeout_s, int64_t copy_slots) {
  CHECK_CUDA_CONTIG(W);
  CHECK_CUDA_CONTIG(Y);
  TORCH_CHECK(copy_slots >= 0 && copy_slots <= 3, "tp2_gemm_allgather_: copy_slots is 0 (choose from the shape), 1, 2 or 3");
  TORCH_CHECK(W.scalar_type() == at::kBFloat16 && Y.scalar_type() == at::kBFloat16 && W.dim() == 2 && Y.dim() == 2, "tp2_gemm_allgather_: bf16 2-D");
  TORCH_CHECK(chunk_flags.scalar_type() == at::kInt && chunk_flags.numel() >= 8 && chunk_counter.scalar_type() == at::kInt && chunk_counter.numel() >= 8, "tp2_gemm_allgather_: int32[8] flags / counters");
  const int64_t N = w_kmajor ? W.size(0) : W.size(1), K = w_kmajor ? W.size(1) : W.size(0);
  TORCH_CHECK(Y.size(1) == N, "tp2_gemm_allgather_: output columns must match the weight");
  ab::TpGemmParams p{};
  p.world = (int)xfull_ptrs.size(); p.rank = (int)rank; p.unit = (int)unit; p.max_units = (int)max_units; p.epoch = (int)epoch;
  p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  fill_ptrs(p.flags, flag_ptrs); fill_ptrs(p.x_full, xfull_ptrs);
  p.chunk_flags = chunk_flags.data_ptr<int>(); p.chunk_counter = chunk_counter.data_ptr<int>();
  p.copy_slots = (int)copy_slots;
  const c10::cuda::CUDAGuard guard(W.device());
  count();
  const int rc = ab::gemm_allgather2(W.data_ptr(), w_kmajor, Y.data_ptr(), (int)Y.size(0), (int)N, (int)K, Y.stride(0), p,
                                     status_tensor(W.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_allgather2 launch failed with code ", rc, " (-2: M must be a multiple of world*256, N of 32, K of 8)");
}

void tp2_gemm_reducescatter_(const Tensor& X, const Tensor& W, bool w_kmajor, std::vector<int64_t> part_ptrs, Tensor& gathered,
                             Tensor& out, std::vector<int64_t> flag_ptrs, Tensor& tile_counter, Tensor& pull_counter,
                             int64_t rank, int64_t unit, int64_t max_units, int64_t epoch, double timeout_s, int64_t phase,
                             int64_t copy_slots) {
  TORCH_CHECK(copy_slots >= 0 && copy_slots <= 3, "tp2_gemm_reducescatter_: copy_slots is 0 (choose from the shape), 1, 2 or 3");
  CHECK_CUDA_CONTIG(X);
  CHECK_CUDA_CONTIG(W);
  CHECK_CUDA_CONTIG(out);
  CHECK_CUDA_CONTIG(gathered);
  TORCH_CHECK(X.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 &&
              gathered.scalar_type() == at::kBFloat16, "tp2_gemm_reducescatter_: bf16");
  const int64_t N = w_kmajor ? W.size(0) : W.size(1), K = w_kmajor ? W.size(1) : W.size(0);
  TORCH_CHECK(X.dim() == 2 && W.dim() == 2 && X.size(1) == K, "tp2_gemm_reducescatter_: inner dimensions differ");
  TORCH_CHECK(tile_counter.scalar_type() == at::kInt && tile_counter.numel() >= 8 && pull_counter.scalar_type() == at::kInt &&
              pull_counter.numel() >= 1, "tp2_gemm_reducescatter_: int32 counters");
  ab::TpGemmParams p{};
  p.world = (int)part_ptrs.size(); p.rank = (int)rank; p.unit = (int)unit; p.max_units = (int)max_units; p.epoch = (int)epoch;
  p.fuse_reduce = (int)phase; p.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  TORCH_CHECK(phase >= 0 && phase <= 2, "tp2_gemm_reducescatter_: phase is 0, 1 or 2");
  TORCH_CHECK(out.size(0) * p.world == X.size(0) && out.size(1) == N, "tp2_gemm_reducescatter_: output must be [M/world, N]");
  TORCH_CHECK(gathered.numel() >= X.size(0) * N, "tp2_gemm_reducescatter_: gathered must hold world slots of [M/world, N]");
  fill_ptrs(p.flags, flag_ptrs); fill_ptrs(p.stage, part_ptrs);
  p.rs_out = out.data_ptr(); p.tile_counter = tile_counter.data_ptr<int>();
  p.gathered = gathered.data_ptr(); p.pull_counter = pull_counter.data_ptr<int>();
  p.copy_slots = (int)copy_slots;
  const c10::cuda::CUDAGuard guard(X.device());
  count();
  const int rc = ab::gemm_reducescatter2(X.data_ptr(), W.data_ptr(), w_kmajor, (int)X.size(0), (int)N, (int)K, p,
                                         status_tensor(X.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_reducescatter2 launch failed with code ", rc, " (-2: M must be a multiple of world*256, N of 32, K of 8)");
}

void tp_reduce_(const Tensor& stage, Tensor& out, int64_t world) {
  CHECK_CUDA_CONTIG(stage);
  CHECK_CUDA_CONTIG(out);
  TORCH_CHECK(stage.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 && stage.numel() == out.numel() * world, "tp_reduce_: stage must hold `world` slots of out");
  const c10::cuda::CUDAGuard guard(out.device());
  count();
  TORCH_CHECK(ab::tp_reduce(stage.data_ptr(), out.data_ptr(), out.size(0), (int)out.size(1), (int)world, stream()) == 0, "tp_reduce launch failed");
}

// ---- fp8
bool is_e5m2(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kFloat8_e4m3fn || t.scalar_type() == at::kFloat8_e5m2, "expected a float8 tensor");
  return t.scalar_type() == at::kFloat8_e5m2;
}

std::tuple<Tensor, Tensor, Tensor> fp8_quantize(const Tensor& x, const Tensor& scale, bool e5m2, bool with_transpose) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1, "fp8_quantize: 2-D bf16 input with unit column stride");
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == 1, "fp8_quantize: scale is one fp32 value on the device");
  const c10::cuda::CUDAGuard guard(x.device());
  const auto dt = e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn;
  Tensor q = at::empty({x.size(0), x.size(1)}, x.options().dtype(dt));
  Tensor qt = with_transpose ? at::empty({x.size(1), x.size(0)}, x.options().dtype(dt)) : at::empty({0}, x.options().dtype(dt));
  Tensor amax = at::zeros({1}, x.options().dtype(at::kFloat));
  count();
  const int rc = ab::fp8_quantize(x.data_ptr(), q.data_ptr(), with_transpose ? qt.data_ptr() : nullptr, scale.data_ptr<float>(),
                                  amax.data_ptr<float>(), (int)x.size(0), (int)x.size(1), x.stride(0), e5m2, stream());
  TORCH_CHECK(rc == 0, "fp8_quantize launch failed with code ", rc);
  return {q, qt, amax};
}

Tensor fp8_gemm(const Tensor& a, const Tensor& b, const Tensor& scale_a, const Tensor& scale_b, const c10::optional<Tensor>& bias) {
  CHECK_CUDA_CONTIG(a);
  CHECK_CUDA_CONTIG(b);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "fp8_gemm: A [M,K], B [N,K]");
  TORCH_CHECK(a.size(1) % 16 == 0, "fp8_gemm: K must be a multiple of 16");
  TORCH_CHECK(scale_a.scalar_type() == at::kFloat && scale_b.scalar_type() == at::kFloat && scale_a.numel() == 1 && scale_b.numel() == 1, "fp8_gemm: per-tensor fp32 scales");
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == b.size(0) && bias->is_contiguous(), "fp8_gemm: bf16 bias [N]");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty({a.size(0), b.size(0)}, a.options().dtype(at::kBFloat16));
  count();
  const int rc = ab::gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), scale_a.data_ptr<float>(), scale_b.data_ptr<float>(),
                              bias.has_value() ? bias->data_ptr() : nullptr, (int)a.size(0), (int)b.size(0), (int)a.size(1),
                              out.stride(0), is_e5m2(a), is_e5m2(b), status_tensor(a.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_fp8 launch failed with code ", rc);
  return out;
}

// ---- block-scaled fp8
std::tuple<Tensor, Tensor> fp8_quantize_block(const Tensor& x, bool weight) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1 && x.size(1) % 128 == 0,
              "fp8_quantize_block: bf16 [rows, cols] with cols a multiple of 128");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), cols = x.size(1);
  Tensor q = at::empty({rows, cols}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor s = weight ? at::empty({(rows + 127) / 128, cols / 128}, x.options().dtype(at::kFloat))
                    : at::empty({cols / 128, rows}, x.options().dtype(at::kFloat));
  count();
  const int rc = weight ? ab::fp8_quantize_weight_block(x.data_ptr(), q.data_ptr(), s.data_ptr<float>(), (int)rows, (int)cols, x.stride(0), stream())
                        : ab::fp8_quantize_act_block(x.data_ptr(), q.data_ptr(), s.data_ptr<float>(), (int)rows, (int)cols, x.stride(0), stream());
  TORCH_CHECK(rc == 0, "fp8_quantize_block failed with code ", rc);
  return {q, s};
}

Tensor fp8_gemm_block(const Tensor& a, const Tensor& sa_t, const Tensor& b, const Tensor& sb, const c10::optional<Tensor>& bias) {
  CHECK_CUDA_CONTIG(a);
  CHECK_CUDA_CONTIG(b);
  TORCH_CHECK(a.scalar_type() == at::kFloat8_e4m3fn && b.scalar_type() == at::kFloat8_e4m3fn && a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "fp8_gemm_block: E4M3 A [M,K], B [N,K]");
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  TORCH_CHECK(K % 128 == 0, "fp8_gemm_block: K must be a multiple of 128");
  TORCH_CHECK(sa_t.is_cuda() && sa_t.scalar_type() == at::kFloat && sa_t.is_contiguous() && sa_t.dim() == 2 && sa_t.size(0) == K / 128 && sa_t.size(1) == M, "fp8_gemm_block: sa_t fp32 [K/128, M]");
  TORCH_CHECK(sb.is_cuda() && sb.scalar_type() == at::kFloat && sb.is_contiguous() && sb.dim() == 2 && sb.size(0) == (N + 127) / 128 && sb.size(1) == K / 128, "fp8_gemm_block: sb fp32 [ceil(N/128), K/128]");
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "fp8_gemm_block: bf16 bias [N]");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty({M, N}, a.options().dtype(at::kBFloat16));
  count();
  const int rc = ab::gemm_fp8_block(a.data_ptr(), b.data_ptr(), out.data_ptr(), sa_t.data_ptr<float>(), sb.data_ptr<float>(),
                                    bias.has_value() ? bias->data_ptr() : nullptr, (int)M, (int)N, (int)K, out.stride(0),
                                    status_tensor(a.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_fp8_block launch failed with code ", rc);
  return out;
}

// ---- sampling
std::tuple<Tensor, Tensor, Tensor> sample_rows(const Tensor& logits, const Tensor& temps, const c10::optional<Tensor>& top_k,
                                               const c10::optional<Tensor>& top_p, const c10::optional<Tensor>& penalty,
                                               const c10::optional<Tensor>& hist, const c10::optional<Tensor>& hist_mask,
                                               bool all_greedy, int64_t seed, int64_t offset) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1 &&
                  (logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat), "sample_rows: bf16 / fp32 logits [rows, V]");
  const int64_t rows = logits.size(0), V = logits.size(1);
  auto f32 = [&](const Tensor& t) { return t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == rows; };
  TORCH_CHECK(f32(temps), "sample_rows: fp32 temperatures [rows]");
  if (top_k.has_value()) TORCH_CHECK(top_k->is_cuda() && top_k->scalar_type() == at::kInt && top_k->is_contiguous() && top_k->numel() == rows, "sample_rows: int32 top_k [rows]");
  if (top_p.has_value()) TORCH_CHECK(f32(*top_p), "sample_rows: fp32 top_p [rows]");
  if (penalty.has_value()) TORCH_CHECK(f32(*penalty), "sample_rows: fp32 penalty [rows]");
  int hist_len = 0;
  if (hist.has_value()) {
    TORCH_CHECK(hist->is_cuda() && hist->scalar_type() == at::kLong && hist->is_contiguous() && hist->dim() == 2 && hist->size(0) == rows, "sample_rows: int64 history [rows, H]");
    hist_len = (int)hist->size(1);
    if (hist_mask.has_value()) TORCH_CHECK(hist_mask->is_cuda() && hist_mask->scalar_type() == at::kBool && hist_mask->is_contiguous() && hist_mask->sizes() == hist->sizes(), "sample_rows: bool history mask [rows, H]");
  }
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor tok = at::empty({rows}, logits.options().dtype(at::kLong));
  Tensor logp = at::empty({rows}, logits.options().dtype(at::kFloat));
  Tensor work = all_greedy ? at::empty({0}, logp.options()) : at::empty({rows, V}, logp.options());
  count();
  const int rc = ab::sample_rows(logits.data_ptr(), logits.scalar_type() == at::kBFloat16, logits.stride(0), all_greedy ? nullptr : work.data_ptr<float>(),
                                 temps.data_ptr<float>(), top_k.has_value() ? top_k->data_ptr<int>() : nullptr,
                                 top_p.has_value() ? top_p->data_ptr<float>() : nullptr, penalty.has_value() ? penalty->data_ptr<float>() : nullptr,
                                 hist.has_value() ? reinterpret_cast<const long long*>(hist->data_ptr<int64_t>()) : nullptr,
                                 hist.has_value() && hist_mask.has_value() ? hist_mask->data_ptr<bool>() : nullptr, hist_len, (int)rows, (int)V,
                                 all_greedy, (unsigned long long)seed, (unsigned long long)offset,
                                 reinterpret_cast<long long*>(tok.data_ptr<int64_t>()), logp.data_ptr<float>(), stream());
  TORCH_CHECK(rc == 0, "sample_rows launch failed with code ", rc);
  return {tok, logp, work};
}

// ---- int8: per-row symmetric quantisation and the kind::i8 GEMM
std::tuple<Tensor, Tensor> int8_quantize_rows(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1, "int8_quantize_rows: bf16 [rows, cols]");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor q = at::empty({x.size(0), x.size(1)}, x.options().dtype(at::kChar));
  Tensor scale = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  count();
  const int rc = ab::int8_quantize_rows(x.data_ptr(), q.data_ptr(), scale.data_ptr<float>(), (int)x.size(0), (int)x.size(1), x.stride(0), stream());
  TORCH_CHECK(rc == 0, "int8_quantize_rows: columns and row stride must be multiples of 8, 16-byte aligned input (code ", rc, ")");
  return {q, scale};
}

Tensor int8_gemm(const Tensor& a, const Tensor& b, const Tensor& row_scale, const Tensor& col_scale, const c10::optional<Tensor>& bias) {
  CHECK_CUDA_CONTIG(a);
  CHECK_CUDA_CONTIG(b);
  TORCH_CHECK(a.scalar_type() == at::kChar && b.scalar_type() == at::kChar && a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "int8_gemm: int8 A [M,K], B [N,K]");
  TORCH_CHECK(a.size(1) % 16 == 0, "int8_gemm: K must be a multiple of 16");
  TORCH_CHECK(row_scale.is_cuda() && row_scale.scalar_type() == at::kFloat && row_scale.is_contiguous() && row_scale.numel() == a.size(0) &&
                  col_scale.is_cuda() && col_scale.scalar_type() == at::kFloat && col_scale.is_contiguous() && col_scale.numel() == b.size(0),
              "int8_gemm: fp32 row_scale [M], col_scale [N]");
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == b.size(0) && bias->is_contiguous(), "int8_gemm: bf16 bias [N]");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty({a.size(0), b.size(0)}, a.options().dtype(at::kBFloat16));
  count();
  const int rc = ab::gemm_int8(a.data_ptr(), b.data_ptr(), out.data_ptr(), row_scale.data_ptr<float>(), col_scale.data_ptr<float>(),
                               bias.has_value() ? bias->data_ptr() : nullptr, (int)a.size(0), (int)b.size(0), (int)a.size(1),
                               out.stride(0), status_tensor(a.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_int8 launch failed with code ", rc);
  return out;
}

// ---- mixture of experts
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> moe_router(const Tensor& logits, int64_t k, bool renorm) {
  CHECK_CUDA_CONTIG(logits);
  TORCH_CHECK(logits.dim() == 2, "moe_router: logits [tokens, experts]");
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  Tensor probs = at::empty_like(logits);
  Tensor idx = at::empty({T, k}, logits.options().dtype(at::kLong));
  Tensor w = at::empty({T, k}, logits.options());
  Tensor counts = at::zeros({E}, logits.options().dtype(at::kInt));
  Tensor psum = at::zeros({E}, logits.options().dtype(at::kFloat));
  count();
  const int rc = ab::moe_router(logits.data_ptr(), probs.data_ptr(), reinterpret_cast<long long*>(idx.data_ptr<int64_t>()), w.data_ptr(),
                                counts.data_ptr<int>(), psum.data_ptr<float>(), T, (int)E, (int)k, renorm, is_bf16(logits), stream());
  TORCH_CHECK(rc == 0, "moe_router: experts <= 256 and top-k <= 8 (code ", rc, ")");
  return {probs, idx, w, counts, psum};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> moe_plan(const Tensor& counts, int64_t max_tiles) {
  CHECK_CUDA_CONTIG(counts);
  TORCH_CHECK(counts.scalar_type() == at::kInt, "moe_plan: int32 counts");
  const c10::cuda::CUDAGuard guard(counts.device());
  const int64_t E = counts.numel();
  Tensor offsets = at::empty({E + 1}, counts.options()), tile_expert = at::empty({max_tiles}, counts.options());
  Tensor cursors = at::empty({E}, counts.options()), total = at::empty({1}, counts.options());
  count();
  TORCH_CHECK(ab::moe_plan(counts.data_ptr<int>(), offsets.data_ptr<int>(), tile_expert.data_ptr<int>(), cursors.data_ptr<int>(),
                           total.data_ptr<int>(), (int)E, (int)max_tiles, stream()) == 0, "moe_plan launch failed");
  return {offsets, tile_expert, cursors, total};
}

std::tuple<Tensor, Tensor> moe_permute(const Tensor& x, const Tensor& idx, const Tensor& counts, const Tensor& offsets, Tensor& cursors,
                                       int64_t max_rows) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(idx);
  TORCH_CHECK(x.dim() == 2 && idx.dim() == 2 && idx.scalar_type() == at::kLong && idx.size(0) == x.size(0), "moe_permute: x [T,D], idx [T,K] int64");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor sorted = at::empty({max_rows, x.size(1)}, x.options());
  Tensor slot_of = at::empty({idx.size(0), idx.size(1)}, x.options().dtype(at::kInt));
  count(2);
  const int rc = ab::moe_permute(x.data_ptr(), reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), counts.data_ptr<int>(),
                                 offsets.data_ptr<int>(), cursors.data_ptr<int>(), sorted.data_ptr(), slot_of.data_ptr<int>(), x.size(0),
                                 (int)idx.size(1), (int)x.size(1), (int)counts.numel(), is_bf16(x), stream());
  TORCH_CHECK(rc == 0, "moe_permute: hidden size must be a multiple of 8 (code ", rc, ")");
  return {sorted, slot_of};
}

Tensor moe_combine(const Tensor& y, const Tensor& slot_of, const c10::optional<Tensor>& weights) {
  CHECK_CUDA_CONTIG(y);
  CHECK_CUDA_CONTIG(slot_of);
  const c10::cuda::CUDAGuard guard(y.device());
  Tensor out = at::empty({slot_of.size(0), y.size(1)}, y.options());
  count();
  const int rc = ab::moe_combine(y.data_ptr(), slot_of.data_ptr<int>(), weights.has_value() ? weights->data_ptr() : nullptr, out.data_ptr(),
                                 slot_of.size(0), (int)slot_of.size(1), (int)y.size(1), is_bf16(y), stream());
  TORCH_CHECK(rc == 0, "moe_combine launch failed with code ", rc);
  return out;
}

std::tuple<Tensor, Tensor> moe_combine_bwd(const Tensor& dout, const Tensor& y, const Tensor& slot_of, const Tensor& weights) {
  CHECK_CUDA_CONTIG(dout);
  CHECK_CUDA_CONTIG(y);
  const c10::cuda::CUDAGuard guard(y.device());
  Tensor dy = at::zeros_like(y);  // padding rows must stay zero: they enter the expert weight gradients
  Tensor dw = at::empty({slot_of.size(0), slot_of.size(1)}, y.options().dtype(at::kFloat));
  count();
  const int rc = ab::moe_combine_bwd(dout.data_ptr(), y.data_ptr(), slot_of.data_ptr<int>(), weights.data_ptr(), dy.data_ptr(),
                                     dw.data_ptr<float>(), slot_of.size(0), (int)slot_of.size(1), (int)y.size(1), is_bf16(y), stream());
  TORCH_CHECK(rc == 0, "moe_combine_bwd launch failed with code ", rc);
  return {dy, dw};
}

// x [R, K] sorted rows; w stacked [E, N, K] (w_kmajor) or consumed as [E, Kc, N'] (MN-major: contraction over dim 1)
Tensor grouped_gemm_rows(const Tensor& x, const Tensor& w, bool w_kmajor, const Tensor& tile_expert) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(w);
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && w.dim() == 3 && x.dim() == 2, "grouped_gemm_rows: bf16 x [R,K], w [E,a,b]");
  const int64_t E = w.size(0), K = x.size(1);
  const int64_t N = w_kmajor ? w.size(1) : w.size(2);
  TORCH_CHECK((w_kmajor ? w.size(2) : w.size(1)) == K, "grouped_gemm_rows: inner dimensions differ");
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.numel() * 128 >= x.size(0), "grouped_gemm_rows: tile map too short");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty({x.size(0), N}, x.options());
  ab::GroupedParams g{};
  g.tile_expert = tile_expert.data_ptr<int>();
  g.b_rows_per_expert = (int)w.size(1);
  g.b_row_offset = 0;
  g.E = (int)E;
  count();
  const int rc = ab::gemm_grouped_rows(x.data_ptr(), w.data_ptr(), y.data_ptr(), (int)x.size(0), (int)N, (int)K, x.stride(0), E * w.size(1),
                                       w.size(2), y.stride(0), w_kmajor, g, status_tensor(x.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_grouped_rows launch failed with code ", rc, " (-2: rows not a multiple of 128, -3: contraction not a multiple of 64)");
  return y;
}

// ---- expert parallel: routing exchange and the grouped GEMM with gather / scatter over peer memory
void ep_push_counts(const Tensor& counts_local, std::vector<int64_t> counts_all_ptrs, Tensor& row_peer_local,
                    std::vector<int64_t> flag_ptrs, int64_t rank, int64_t unit, int64_t max_units, int64_t epoch) {
  TORCH_CHECK(counts_local.is_cuda() && counts_local.scalar_type() == at::kInt && row_peer_local.scalar_type() == at::kInt, "ep_push_counts: int32 tensors");
  const int world = (int)counts_all_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && (int)flag_ptrs.size() == world, "ep_push_counts: one pointer per rank");
  void* ca[8]; void* fl[8];
  for (int i = 0; i < world; ++i) ca[i] = reinterpret_cast<void*>(counts_all_ptrs[i]), fl[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  const c10::cuda::CUDAGuard guard(counts_local.device());
  count();
  const int rc = ab::ep_push_counts(counts_local.data_ptr<int>(), (int)counts_local.numel(), ca, row_peer_local.data_ptr<int>(),
                                    (int)row_peer_local.numel(), fl, world, (int)rank, (int)unit, (int)max_units, (int)epoch, stream());
  TORCH_CHECK(rc == 0, "ep_push_counts: experts must divide evenly over <= 8 ranks, <= 256 experts, row table a multiple of 128 (code ", rc, ")");
}

std::tuple<Tensor, Tensor, Tensor> ep_plan(const Tensor& idx, const Tensor& counts_all_local, std::vector<int64_t> row_peer_ptrs,
                                           int64_t n_experts, int64_t r_cap, std::vector<int64_t> flag_ptrs, int64_t rank,
                                           int64_t wait_unit, int64_t signal_unit, int64_t max_units, int64_t epoch, double timeout_s) {
  CHECK_CUDA_CONTIG(idx);
  TORCH_CHECK(idx.scalar_type() == at::kLong && counts_all_local.scalar_type() == at::kInt, "ep_plan: idx int64, counts int32");
  const int world = (int)row_peer_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && (int)flag_ptrs.size() == world && counts_all_local.numel() >= world * n_experts, "ep_plan: one pointer per rank");
  void* rp[8]; void* fl[8];
  for (int i = 0; i < world; ++i) rp[i] = reinterpret_cast<void*>(row_peer_ptrs[i]), fl[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  const c10::cuda::CUDAGuard guard(idx.device());
  auto io = idx.options().dtype(at::kInt);
  Tensor offsets = at::zeros({n_experts / world + 1}, io), tile_expert = at::full({r_cap / 128}, -1, io), total = at::zeros({1}, io);
  count();
  const int rc = ab::ep_plan(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), idx.numel(), counts_all_local.data_ptr<int>(), rp,
                             offsets.data_ptr<int>(), tile_expert.data_ptr<int>(), total.data_ptr<int>(), (int)n_experts, (int)r_cap, fl,
                             world, (int)rank, (int)wait_unit, (int)signal_unit, (int)max_units, (int)epoch,
                             (unsigned long long)(timeout_s * 1e9), status_tensor(idx.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "ep_plan launch failed with code ", rc);
  return {offsets, tile_expert, total};
}

// Rows mode with the sorted rows pulled from (src_ptrs) or the output rows pushed to (dst_ptrs) peer memory.
// Gather: `x` is the local sorted buffer the rows land in (its contents on entry do not matter).  Scatter: the result
// has no local copy and an empty tensor is returned.
Tensor grouped_gemm_rows_ep(Tensor& x, const Tensor& w, bool w_kmajor, const Tensor& tile_expert, const Tensor& row_peer, int64_t rank,
                            std::vector<int64_t> src_ptrs, int64_t src_div, const c10::optional<Tensor>& tile_flags, int64_t n_copy_ctas,
                            std::vector<int64_t> dst_ptrs, const c10::optional<Tensor>& done_counter, std::vector<int64_t> flag_ptrs,
                            int64_t announce_unit, int64_t wait_unit, int64_t signal_unit, int64_t max_units, int64_t epoch,
                            double timeout_s) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(w);
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && w.dim() == 3 && x.dim() == 2, "grouped_gemm_rows_ep: bf16 x [R,K], w [E,a,b]");
  const int64_t E = w.size(0), K = x.size(1);
  const int64_t N = w_kmajor ? w.size(1) : w.size(2);
  TORCH_CHECK((w_kmajor ? w.size(2) : w.size(1)) == K, "grouped_gemm_rows_ep: inner dimensions differ");
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_expert.numel() * 128 >= x.size(0), "grouped_gemm_rows_ep: tile map too short");
  TORCH_CHECK(row_peer.is_cuda() && row_peer.scalar_type() == at::kInt && row_peer.numel() >= x.size(0), "grouped_gemm_rows_ep: row table too short");
  const bool gather = !src_ptrs.empty(), scatter = !dst_ptrs.empty();
  TORCH_CHECK(gather != scatter, "grouped_gemm_rows_ep: exactly one of gather / scatter");
  const int world = (int)flag_ptrs.size();
  TORCH_CHECK(world >= 2 && world <= 8, "grouped_gemm_rows_ep: 2..8 ranks");
  ab::EpRows ep;
  ep.world = world, ep.rank = (int)rank, ep.row_peer = row_peer.data_ptr<int>();
  ep.announce_unit = (int)announce_unit, ep.wait_unit = (int)wait_unit, ep.signal_unit = (int)signal_unit;
  ep.max_units = (int)max_units, ep.epoch = (int)epoch, ep.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  for (int i = 0; i < world; ++i) ep.flags[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  if (gather) {
    TORCH_CHECK((int)src_ptrs.size() == world && tile_flags.has_value() && tile_flags->scalar_type() == at::kInt && tile_flags->numel() * 128 >= x.size(0), "grouped_gemm_rows_ep: gather needs a source per rank and int32 tile flags");
    for (int i = 0; i < world; ++i) ep.src[i] = reinterpret_cast<const void*>(src_ptrs[i]);
    ep.src_div = (int)src_div, ep.tile_flags = tile_flags->data_ptr<int>(), ep.n_copy_ctas = (int)n_copy_ctas;
  } else {
    TORCH_CHECK((int)dst_ptrs.size() == world && done_counter.has_value() && done_counter->scalar_type() == at::kInt && done_counter->numel() >= 1, "grouped_gemm_rows_ep: scatter needs a destination per rank and an int32 counter");
    for (int i = 0; i < world; ++i) ep.dst[i] = reinterpret_cast<void*>(dst_ptrs[i]);
    ep.done_counter = done_counter->data_ptr<int>();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor y = scatter ? at::empty({0}, x.options()) : at::empty({x.size(0), N}, x.options());
  ab::GroupedParams g{};
  g.tile_expert = tile_expert.data_ptr<int>();
  g.b_rows_per_expert = (int)w.size(1);
  g.b_row_offset = 0;
  g.E = (int)E;
  count();
  const int rc = ab::gemm_grouped_rows(x.data_ptr(), w.data_ptr(), scatter ? nullptr : y.data_ptr(), (int)x.size(0), (int)N, (int)K,
                                       x.stride(0), E * w.size(1), w.size(2), N, w_kmajor, g, status_tensor(x.device()).data_ptr<int>(),
                                       stream(), &ep);
  TORCH_CHECK(rc == 0, "grouped_gemm_rows_ep launch failed with code ", rc);
  return y;
}

// dW [E, N, K] = per-expert dY_e^T X_e over the padded segments given by offsets [E+1]
Tensor grouped_gemm_wgrad(const Tensor& dy, const Tensor& x, const Tensor& offsets, bool out_f32) {
  CHECK_CUDA_CONTIG(dy);
  CHECK_CUDA_CONTIG(x);
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16 && dy.size(0) == x.size(0), "grouped_gemm_wgrad: bf16 [R,N], [R,K]");
  const int64_t E = offsets.numel() - 1, N = dy.size(1), K = x.size(1);
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor dw = at::empty({E, N, K}, x.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  ab::GroupedParams g{};
  g.offsets = offsets.data_ptr<int>();
  g.d_expert_stride = N * K;
  g.E = (int)E;
  count();
  const int rc = ab::gemm_grouped_wgrad(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), (int)x.size(0), (int)N, (int)K, dy.stride(0), x.stride(0), K,
                                        out_f32, false, g, status_tensor(x.device()).data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_grouped_wgrad launch failed with code ", rc);
  return dw;
}

void kernel_status_reset(const Tensor& like) { status_tensor(like.device()).zero_(); }

}  // namespace

TORCH_LIBRARY(astrai_b200, m) {
  m.def("rmsnorm_fwd(Tensor x, Tensor w, float eps) -> (Tensor, Tensor)", &rmsnorm_fwd);
  m.def("rmsnorm_bwd(Tensor g, Tensor x, Tensor w, Tensor rstd) -> (Tensor, Tensor)", &rmsnorm_bwd);
  m.def("add_rmsnorm_fwd(Tensor x, Tensor res, Tensor w, float eps) -> (Tensor, Tensor, Tensor)", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd_add(Tensor g, Tensor x, Tensor w, Tensor rstd, Tensor gres) -> (Tensor, Tensor)", &rmsnorm_bwd_add);
  m.def("rope(Tensor x, Tensor(a!) out, Tensor freqs, bool inverse) -> ()", &rope);
  m.def("swiglu_fwd(Tensor gate, Tensor up) -> Tensor", &swiglu_fwd);
  m.def("swiglu_bwd(Tensor dy, Tensor gate, Tensor up) -> Tensor", &swiglu_bwd);
  m.def("embedding_fwd(Tensor ids, Tensor table) -> Tensor", &embedding_fwd);
  m.def("embedding_bwd_(Tensor ids, Tensor g, Tensor(a!) grad_table) -> ()", &embedding_bwd_);
  m.def("embedding_bwd_sorted_(Tensor sorted_ids, Tensor perm, Tensor g, Tensor(a!) grad_table) -> ()", &embedding_bwd_sorted_);
  m.def("ce_rows(Tensor(a!) logits, Tensor targets, float smoothing, int ignore_index, Tensor? grad_scale, bool in_place_grad) -> (Tensor, Tensor)", &ce_rows);
  m.def("logprob_bwd_(Tensor(a!) logits, Tensor targets, Tensor logprob, Tensor g_rows) -> ()", &logprob_bwd_);
  m.def("sumsq_(Tensor x, Tensor(a!) out) -> ()", &sumsq_);
  m.def("clip_coef_(Tensor sumsq, float max_norm, float pre_scale, Tensor(a!) coef, Tensor(b!) norm) -> ()", &clip_coef_);
  m.def("adamw_(Tensor(a!) p, Tensor? master, Tensor(b!) g, Tensor(c!) m, Tensor(d!) v, float lr, float b1, float b2, float eps, float wd, int step, Tensor? gscale, bool zero_grad) -> ()", &adamw_);
  m.def("axpy_f32_(Tensor(a!) dst, Tensor src, float alpha) -> ()", &axpy_f32_);
  m.def("kernel_status(Tensor like) -> Tensor", &kernel_status);
  m.def("launch_count() -> int", &launch_count);
  m.def("kv_append_(Tensor k_new, Tensor v_new, Tensor(a!) k_buf, Tensor(b!) v_buf, Tensor loc) -> ()", &kv_append_);
  m.def("paged_decode_splits(int batch, int n_kv_heads, int max_len, int max_splits) -> int", &paged_decode_splits);
  m.def("paged_decode_(Tensor q, Tensor k_buf, Tensor v_buf, Tensor req_to_token, Tensor req_pool_indices, Tensor seq_lens, float scale, int splits, Tensor(a!) o_part, Tensor(b!) ml_part, Tensor(c!) counters, Tensor(d!) out) -> ()", &paged_decode_);
  m.def("paged_decode_append_(Tensor q, Tensor k_new, Tensor v_new, Tensor(a!) k_buf, Tensor(b!) v_buf, Tensor req_to_token, Tensor req_pool_indices, Tensor seq_lens, float scale, int splits, Tensor(c!) o_part, Tensor(d!) ml_part, Tensor(e!) counters, Tensor(f!) out) -> ()", &paged_decode_append_);
  m.def("fsdp_reduce_scatter_(int[] grad_ptrs, int mc_ptr, int[] flag_ptrs, int rank, int shard_off, Tensor(a!) out, Tensor(b!) sumsq, int unit, int max_units, int epoch, float timeout_s, int max_ctas) -> ()", &fsdp_reduce_scatter_);
  m.def("fsdp_adamw_allgather_(int[] param_ptrs, int mc_ptr, int[] flag_ptrs, int rank, int shard_off, Tensor? master, Tensor g, Tensor(a!) m, Tensor(b!) v, float lr, float b1, float b2, float eps, float wd, int step, Tensor? gscale, int unit, int max_units, int epoch, Tensor(c!) block_counter, int max_ctas) -> ()", &fsdp_adamw_allgather_);
  m.def("comm_wait_flags_(Tensor local_flags, int kind, int world, int skip_rank, int unit, int max_units, int epoch, float timeout_s) -> ()", &comm_wait_flags_);
  m.def("kernel_status_reset(Tensor like) -> ()", &kernel_status_reset);
  m.def("flash_fwd(Tensor q, Tensor k, Tensor v, Tensor? cu_q, Tensor? cu_k, int batch, int sq, int sk, int max_q, bool causal, float scale) -> (Tensor, Tensor)", &flash_fwd);
  m.def("flash_fwd_paged(Tensor q, Tensor k_pool, Tensor v_pool, Tensor cu_q, Tensor cu_k, Tensor table, Tensor rows, int page, int max_q, bool causal, float scale) -> Tensor", &flash_fwd_paged);
  m.def("flash_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor dout, Tensor lse, Tensor? cu_q, Tensor? cu_k, int batch, int sq, int sk, int max_q, int max_k, bool causal, float scale) -> (Tensor, Tensor, Tensor)", &flash_bwd);
  m.def("cp_flash_fwd(Tensor q, Tensor k_full, Tensor v_full, int batch, int chunk, int world, int rank, float scale, int[] kv_src_ptrs, int[] flag_ptrs, int unit, int max_units, int epoch, int n_copy_ctas, Tensor? chunk_state, float timeout_s) -> (Tensor, Tensor)", &cp_flash_fwd);
  m.def("cp_flash_bwd(Tensor q, Tensor k_full, Tensor v_full, Tensor out, Tensor dout, Tensor lse, int batch, int chunk, int world, int rank, float scale, int[] stage_ptrs, int[] flag_ptrs, int unit, int max_units, int epoch, Tensor? tile_counter, float timeout_s) -> (Tensor, Tensor, Tensor)", &cp_flash_bwd);
  m.def("cp_dkv_reduce(Tensor(a!) dk_local, Tensor(b!) dv_local, int batch, int chunk, int world, int rank, int[] stage_ptrs, int[] flag_ptrs, int unit, int max_units, int epoch, float timeout_s) -> ()", &cp_dkv_reduce);
  m.def("tp_gemm_allgather_(int[] xfull_ptrs, Tensor W, bool w_kmajor, Tensor(a!) Y, int[] flag_ptrs, Tensor(b!) chunk_flags, Tensor(c!) chunk_counter, int rank, int unit, int max_units, int epoch, float timeout_s, int n_copy_ctas) -> ()", &tp_gemm_allgather_);
  m.def("tp_gemm_reducescatter_(Tensor X, Tensor W, bool w_kmajor, int[] stage_ptrs, Tensor(a!) out, int[] flag_ptrs, Tensor(b!) tile_counter, int rank, int unit, int max_units, int epoch, float timeout_s, bool fuse_reduce) -> ()", &tp_gemm_reducescatter_);
  m.def("tp_reduce_(Tensor stage, Tensor(a!) out, int world) -> ()", &tp_reduce_);
  m.def("tp2_gemm_allgather_(int[] xfull_ptrs, Tensor W, bool w_kmajor, Tensor(a!) Y, int[] flag_ptrs, Tensor(b!) chunk_flags, Tensor(c!) chunk_counter, int rank, int unit, int max_units, int epoch, float timeout_s, int copy_slots=0) -> ()", &tp2_gemm_allgather_);
  m.def("tp2_gemm_reducescatter_(Tensor X, Tensor W, bool w_kmajor, int[] part_ptrs, Tensor(a!) gathered, Tensor(b!) out, int[] flag_ptrs, Tensor(c!) tile_counter, Tensor(d!) pull_counter, int rank, int unit, int max_units, int epoch, float timeout_s, int phase, int copy_slots=0) -> ()", &tp2_gemm_reducescatter_);
  m.def("fp8_quantize(Tensor x, Tensor scale, bool e5m2, bool with_transpose) -> (Tensor, Tensor, Tensor)", &fp8_quantize);
  m.def("fp8_gemm(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, Tensor? bias) -> Tensor", &fp8_gemm);
  m.def("sample_rows(Tensor logits, Tensor temps, Tensor? top_k, Tensor? top_p, Tensor? penalty, Tensor? hist, Tensor? hist_mask, bool all_greedy, int seed, int offset) -> (Tensor, Tensor, Tensor)", &sample_rows);
  m.def("fp8_quantize_block(Tensor x, bool weight) -> (Tensor, Tensor)", &fp8_quantize_block);
  m.def("fp8_gemm_block(Tensor a, Tensor sa_t, Tensor b, Tensor sb, Tensor? bias) -> Tensor", &fp8_gemm_block);
  m.def("int8_quantize_rows(Tensor x) -> (Tensor, Tensor)", &int8_quantize_rows);
  m.def("int8_gemm(Tensor a, Tensor b, Tensor row_scale, Tensor col_scale, Tensor? bias) -> Tensor", &int8_gemm);
  m.def("moe_router(Tensor logits, int k, bool renorm) -> (Tensor, Tensor, Tensor, Tensor, Tensor)", &moe_router);
  m.def("moe_plan(Tensor counts, int max_tiles) -> (Tensor, Tensor, Tensor, Tensor)", &moe_plan);
  m.def("moe_permute(Tensor x, Tensor idx, Tensor counts, Tensor offsets, Tensor(a!) cursors, int max_rows) -> (Tensor, Tensor)", &moe_permute);
  m.def("moe_combine(Tensor y, Tensor slot_of, Tensor? weights) -> Tensor", &moe_combine);
  m.def("moe_combine_bwd(Tensor dout, Tensor y, Tensor slot_of, Tensor weights) -> (Tensor, Tensor)", &moe_combine_bwd);
  m.def("grouped_gemm_rows(Tensor x, Tensor w, bool w_kmajor, Tensor tile_expert) -> Tensor", &grouped_gemm_rows);
  m.def("grouped_gemm_wgrad(Tensor dy, Tensor x, Tensor offsets, bool out_f32) -> Tensor", &grouped_gemm_wgrad);
  m.def("ep_push_counts(Tensor counts_local, int[] counts_all_ptrs, Tensor(a!) row_peer_local, int[] flag_ptrs, int rank, int unit, int max_units, int epoch) -> ()", &ep_push_counts);
  m.def("ep_plan(Tensor idx, Tensor counts_all_local, int[] row_peer_ptrs, int n_experts, int r_cap, int[] flag_ptrs, int rank, int wait_unit, int signal_unit, int max_units, int epoch, float timeout_s) -> (Tensor, Tensor, Tensor)", &ep_plan);
  m.def("grouped_gemm_rows_ep(Tensor(a!) x, Tensor w, bool w_kmajor, Tensor tile_expert, Tensor row_peer, int rank, int[] src_ptrs, int src_div, Tensor? tile_flags, int n_copy_ctas, int[] dst_ptrs, Tensor? done_counter, int[] flag_ptrs, int announce_unit, int wait_unit, int signal_unit, int max_units, int epoch, float timeout_s) -> Tensor", &grouped_gemm_rows_ep);
  m.def("gemm(Tensor A, Tensor B, Tensor? D, bool a_kmajor, bool b_kmajor, bool out_f32, bool accumulate) -> Tensor", &gemm);
}
