// Torch-free check of the tensor-core GEMM family and of prefill attention over a paged pool: links the GEMM sources and
// flash_fwd.cu only, allocates with cudaMalloc and compares every result with CPU fp32 arithmetic on the very operands the
// kernels consumed (the quantised bytes and scales are copied back and decoded on the host, so the comparison isolates
// the matrix product from the rounding of the quantiser).
//   build:  python -m astrai_b200.ops.build --standalone      (writes astrai_b200/ops/build/quant_paged_check)
//   run  :  astrai_b200/ops/build/quant_paged_check            (exit code 0 = every case within tolerance)
// Counterpart of the reference's torch-free fp8 MMA test and paged-attention test
// (csrc/tests/fp8_mma_test.cu, csrc/tests/attn_paged_test.cu:702-870).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <random>
#include <vector>

#include "../launchers.h"

#define CK(x)                                                                                  \
  do {                                                                                         \
    cudaError_t e_ = (x);                                                                      \
    if (e_ != cudaSuccess) {                                                                   \
      std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));         \
      std::exit(2);                                                                            \
    }                                                                                          \
  } while (0)

namespace {

std::mt19937 g_rng(4321);
int g_failures = 0;

std::vector<__nv_bfloat16> random_bf16(size_t n, float scale = 1.f) {
  std::normal_distribution<float> d(0.f, scale);
  std::vector<__nv_bfloat16> v(n);
  for (auto& x : v) x = __float2bfloat16(d(g_rng));
  return v;
}

template <typename T>
T* to_device(const std::vector<T>& h) {
  T* d = nullptr;
  CK(cudaMalloc(&d, std::max<size_t>(h.size(), 1) * sizeof(T)));
  CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}

template <typename T>
T* device_zeros(size_t n) {
  T* d = nullptr;
  CK(cudaMalloc(&d, std::max<size_t>(n, 1) * sizeof(T)));
  CK(cudaMemset(d, 0, std::max<size_t>(n, 1) * sizeof(T)));
  return d;
}

template <typename T>
std::vector<T> to_host(const T* d, size_t n) {
  std::vector<T> h(n);
  CK(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost));
  return h;
}

float f8(uint8_t byte, bool e5m2) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, e5m2 ? __NV_E5M2 : __NV_E4M3);
  return __half2float(__half(h));
}

// max |got - want| / max |want| over a [M, N] result
void report(const char* what, const std::vector<float>& want, const std::vector<float>& got, float tol) {
  float err = 0.f, mx = 1e-20f;
  for (size_t i = 0; i < want.size(); ++i) {
    err = std::max(err, std::fabs(want[i] - got[i]));
    mx = std::max(mx, std::fabs(want[i]));
  }
  const bool ok = std::isfinite(err) && err / mx < tol;
  std::printf("  %-64s rel err %.2e  %s\n", what, err / mx, ok ? "ok" : "FAIL");
  if (!ok) ++g_failures;
}

std::vector<float> bf16_to_float(const std::vector<__nv_bfloat16>& v) {
  std::vector<float> f(v.size());
  for (size_t i = 0; i < v.size(); ++i) f[i] = __bfloat162float(v[i]);
  return f;
}

// want[m, n] = sum_k a[m, k] * b[n, k]
std::vector<float> cpu_nt(const std::vector<float>& a, const std::vector<float>& b, int M, int N, int K) {
  std::vector<float> d((size_t)M * N);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      double s = 0.0;
      const float *pa = &a[(size_t)m * K], *pb = &b[(size_t)n * K];
      for (int k = 0; k < K; ++k) s += (double)pa[k] * pb[k];
      d[(size_t)m * N + n] = (float)s;
    }
  return d;
}

void check_bf16(int M, int N, int K, bool accumulate, int* status) {
  auto a = random_bf16((size_t)M * K), b = random_bf16((size_t)N * K);
  __nv_bfloat16 *da = to_device(a), *db = to_device(b);
  auto want = cpu_nt(bf16_to_float(a), bf16_to_float(b), M, N, K);
  char name[128];
  if (accumulate) {  // fp32 output, D += A B^T on top of a known start (the weight-gradient epilogue)
    std::vector<float> start((size_t)M * N, 0.5f);
    float* dd = to_device(start);
    const int rc = ab::gemm_bf16(da, db, dd, M, N, K, K, K, N, true, true, true, true, status, 0);
    CK(cudaDeviceSynchronize());
    auto got = to_host(dd, (size_t)M * N);
    for (auto& w : want) w += 0.5f;
    std::snprintf(name, sizeof name, "bf16 GEMM %dx%dx%d, fp32 accumulate-into (rc %d)", M, N, K, rc);
    report(name, want, got, 2e-3f);
    CK(cudaFree(dd));
  } else {
    __nv_bfloat16* dd = device_zeros<__nv_bfloat16>((size_t)M * N);
    const int rc = ab::gemm_bf16(da, db, dd, M, N, K, K, K, N, true, true, false, false, status, 0);
    CK(cudaDeviceSynchronize());
    auto got = bf16_to_float(to_host(dd, (size_t)M * N));
    std::snprintf(name, sizeof name, "bf16 GEMM %dx%dx%d, bf16 out (rc %d)", M, N, K, rc);
    report(name, want, got, 1e-2f);
    CK(cudaFree(dd));
  }
  CK(cudaFree(da));
  CK(cudaFree(db));
}

void check_fp8(int M, int N, int K, bool a_e5m2, int* status) {
  auto a = random_bf16((size_t)M * K), b = random_bf16((size_t)N * K);
  __nv_bfloat16 *da = to_device(a), *db = to_device(b);
  uint8_t *qa = device_zeros<uint8_t>((size_t)M * K), *qb = device_zeros<uint8_t>((size_t)N * K);
  const std::vector<float> scales = {4.f / (a_e5m2 ? 57344.f : 448.f), 4.f / 448.f};  // |x| <= ~4 sigma maps onto the format's range
  float* dscale = to_device(scales);
  float* amax = device_zeros<float>(2);
  int rc = ab::fp8_quantize(da, qa, nullptr, dscale, amax, M, K, K, a_e5m2, 0);
  rc |= ab::fp8_quantize(db, qb, nullptr, dscale + 1, amax + 1, N, K, K, false, 0);
  __nv_bfloat16* dd = device_zeros<__nv_bfloat16>((size_t)M * N);
  rc |= ab::gemm_fp8(qa, qb, dd, dscale, dscale + 1, nullptr, M, N, K, N, a_e5m2, false, status, 0);
  CK(cudaDeviceSynchronize());
  auto ha = to_host(qa, (size_t)M * K), hb = to_host(qb, (size_t)N * K);
  std::vector<float> fa(ha.size()), fb(hb.size());
  for (size_t i = 0; i < ha.size(); ++i) fa[i] = f8(ha[i], a_e5m2) * scales[0];
  for (size_t i = 0; i < hb.size(); ++i) fb[i] = f8(hb[i], false) * scales[1];
  auto want = cpu_nt(fa, fb, M, N, K);
  auto got = bf16_to_float(to_host(dd, (size_t)M * N));
  char name[128];
  std::snprintf(name, sizeof name, "fp8 GEMM %dx%dx%d (%s x E4M3, per-tensor scales, rc %d)", M, N, K, a_e5m2 ? "E5M2" : "E4M3", rc);
  report(name, want, got, 1e-2f);
  // the quantiser itself: amax is the largest |x|, and decoding reproduces x to the format's precision
  auto hmax = to_host(amax, 2);
  float ref_amax = 0.f, qerr = 0.f;
  auto af = bf16_to_float(a);
  for (size_t i = 0; i < af.size(); ++i) {
    ref_amax = std::max(ref_amax, std::fabs(af[i]));
    if (std::fabs(af[i]) < 3.5f) qerr = std::max(qerr, std::fabs(fa[i] - af[i]) / std::max(std::fabs(af[i]), 0.05f));
  }
  const bool ok = std::fabs(hmax[0] - ref_amax) < 1e-6f && qerr < (a_e5m2 ? 0.13f : 0.07f);
  std::printf("  %-64s amax %.4f (want %.4f), rel step %.3f  %s\n", "fp8 quantiser", hmax[0], ref_amax, qerr, ok ? "ok" : "FAIL");
  if (!ok) ++g_failures;
  for (void* p : {(void*)da, (void*)db, (void*)qa, (void*)qb, (void*)dscale, (void*)amax, (void*)dd}) CK(cudaFree(p));
}

void check_fp8_block(int M, int N, int K, int* status) {
  auto a = random_bf16((size_t)M * K, 2.f), b = random_bf16((size_t)N * K, 0.05f);
  __nv_bfloat16 *da = to_device(a), *db = to_device(b);
  const int KB = K / 128, NB = (N + 127) / 128;
  uint8_t *qa = device_zeros<uint8_t>((size_t)M * K), *qb = device_zeros<uint8_t>((size_t)N * K);
  float *sa = device_zeros<float>((size_t)KB * M), *sb = device_zeros<float>((size_t)NB * KB);
  int rc = ab::fp8_quantize_act_block(da, qa, sa, M, K, K, 0);
  rc |= ab::fp8_quantize_weight_block(db, qb, sb, N, K, K, 0);
  __nv_bfloat16* dd = device_zeros<__nv_bfloat16>((size_t)M * N);
  rc |= ab::gemm_fp8_block(qa, qb, dd, sa, sb, nullptr, M, N, K, N, status, 0);
  CK(cudaDeviceSynchronize());
  auto ha = to_host(qa, (size_t)M * K), hb = to_host(qb, (size_t)N * K);
  auto hsa = to_host(sa, (size_t)KB * M), hsb = to_host(sb, (size_t)NB * KB);
  std::vector<float> fa(ha.size()), fb(hb.size());
  for (int m = 0; m < M; ++m)
    for (int k = 0; k < K; ++k) fa[(size_t)m * K + k] = f8(ha[(size_t)m * K + k], false) * hsa[(size_t)(k / 128) * M + m];
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) fb[(size_t)n * K + k] = f8(hb[(size_t)n * K + k], false) * hsb[(size_t)(n / 128) * KB + k / 128];
  auto want = cpu_nt(fa, fb, M, N, K);
  auto got = bf16_to_float(to_host(dd, (size_t)M * N));
  char name[128];
  std::snprintf(name, sizeof name, "block-scaled fp8 GEMM %dx%dx%d (1x128 / 128x128 scales, rc %d)", M, N, K, rc);
  report(name, want, got, 1e-2f);
  // and against the unquantised product: the block scales keep the quantisation error at the few-percent level
  auto exact = cpu_nt(bf16_to_float(a), bf16_to_float(b), M, N, K);
  report("  ... against the bf16 operands", exact, got, 6e-2f);
  for (void* p : {(void*)da, (void*)db, (void*)qa, (void*)qb, (void*)sa, (void*)sb, (void*)dd}) CK(cudaFree(p));
}

void check_int8(int M, int N, int K, int* status) {
  auto a = random_bf16((size_t)M * K), b = random_bf16((size_t)N * K, 0.1f);
  __nv_bfloat16 *da = to_device(a), *db = to_device(b);
  int8_t *qa = device_zeros<int8_t>((size_t)M * K), *qb = device_zeros<int8_t>((size_t)N * K);
  float *ra = device_zeros<float>(M), *rb = device_zeros<float>(N);
  int rc = ab::int8_quantize_rows(da, qa, ra, M, K, K, 0);
  rc |= ab::int8_quantize_rows(db, qb, rb, N, K, K, 0);
  __nv_bfloat16* dd = device_zeros<__nv_bfloat16>((size_t)M * N);
  rc |= ab::gemm_int8(qa, qb, dd, ra, rb, nullptr, M, N, K, N, status, 0);
  CK(cudaDeviceSynchronize());
  auto ha = to_host(qa, (size_t)M * K), hb = to_host(qb, (size_t)N * K);
  auto hra = to_host(ra, M), hrb = to_host(rb, N);
  std::vector<float> want((size_t)M * N);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      long long s = 0;  // the kernel's int32 sum is exact, so is this one
      for (int k = 0; k < K; ++k) s += (int)ha[(size_t)m * K + k] * (int)hb[(size_t)n * K + k];
      want[(size_t)m * N + n] = (float)s * hra[m] * hrb[n];
    }
  auto got = bf16_to_float(to_host(dd, (size_t)M * N));
  char name[128];
  std::snprintf(name, sizeof name, "int8 GEMM %dx%dx%d (per-row scales, rc %d)", M, N, K, rc);
  report(name, want, got, 6e-3f);
  for (void* p : {(void*)da, (void*)db, (void*)qa, (void*)qb, (void*)ra, (void*)rb, (void*)dd}) CK(cudaFree(p));
}

// Ragged prefill over a paged pool: request b has kv_len[b] cached + new keys in pages scattered over the pool and q_len[b]
// new queries (lower-right aligned causal mask); the kernel reads the pool through the slot table.
void check_paged_prefill(int page, int Hq, int Hkv, int D, const std::vector<int>& q_len, const std::vector<int>& kv_len, int* status) {
  const int B = (int)q_len.size(), G = Hq / Hkv;
  const int max_ctx = ((*std::max_element(kv_len.begin(), kv_len.end()) + page - 1) / page) * page;
  int pages_needed = 0;
  for (int l : kv_len) pages_needed += (l + page - 1) / page;
  const int n_pages = pages_needed + 7;
  std::vector<int> perm(n_pages);
  std::iota(perm.begin(), perm.end(), 0);
  std::shuffle(perm.begin(), perm.end(), g_rng);
  std::vector<int> table((size_t)(B + 2) * max_ctx, 0), rows(B), cu_q(B + 1, 0), cu_k(B + 1, 0);
  int next = 0;
  for (int b = 0; b < B; ++b) {
    rows[b] = B + 1 - b;  // table rows in an order of their own, as a request pool hands them out
    for (int t = 0; t < kv_len[b]; ++t) {
      if (t % page == 0) ++next;
      table[(size_t)rows[b] * max_ctx + t] = perm[next - 1] * page + t % page;
    }
    cu_q[b + 1] = cu_q[b] + q_len[b];
    cu_k[b + 1] = cu_k[b] + kv_len[b];
  }
  const size_t pool = (size_t)n_pages * page * Hkv * D, nq = (size_t)cu_q[B] * Hq * D;
  auto k = random_bf16(pool), v = random_bf16(pool), q = random_bf16(nq);
  __nv_bfloat16 *dk = to_device(k), *dv = to_device(v), *dq = to_device(q), *dout = device_zeros<__nv_bfloat16>(nq);
  int *dt = to_device(table), *dr = to_device(rows), *dcq = to_device(cu_q), *dck = to_device(cu_k);
  ab::PagedKv pg;
  pg.table = dt, pg.rows = dr, pg.stride = max_ctx, pg.page = page;
  const float scale = 1.f / std::sqrt((float)D);
  const int max_q = *std::max_element(q_len.begin(), q_len.end());
  const int rc = ab::flash_fwd(dq, dk, dv, dout, nullptr, dcq, dck, B, 0, 0, max_q, cu_q[B], (long long)n_pages * page, Hq, Hkv, D,
                               (long long)Hq * D, (long long)Hkv * D, (long long)Hkv * D, (long long)Hq * D, scale, true, status, 0,
                               nullptr, &pg);
  CK(cudaDeviceSynchronize());
  auto got = bf16_to_float(to_host(dout, nq));
  std::vector<float> want(nq, 0.f), p;
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < q_len[b]; ++i)
      for (int h = 0; h < Hq; ++h) {
        const int limit = i + kv_len[b] - q_len[b] + 1, kvh = h / G;
        const __nv_bfloat16* qr = &q[((size_t)(cu_q[b] + i) * Hq + h) * D];
        p.assign(limit, 0.f);
        float mx = -INFINITY;
        for (int j = 0; j < limit; ++j) {
          const __nv_bfloat16* kr = &k[((size_t)table[(size_t)rows[b] * max_ctx + j] * Hkv + kvh) * D];
          float s = 0.f;
          for (int d = 0; d < D; ++d) s += __bfloat162float(qr[d]) * __bfloat162float(kr[d]);
          p[j] = s * scale;
          mx = std::max(mx, p[j]);
        }
        float den = 0.f;
        for (int j = 0; j < limit; ++j) den += (p[j] = std::exp(p[j] - mx));
        float* o = &want[((size_t)(cu_q[b] + i) * Hq + h) * D];
        for (int j = 0; j < limit; ++j) {
          const __nv_bfloat16* vr = &v[((size_t)table[(size_t)rows[b] * max_ctx + j] * Hkv + kvh) * D];
          const float w = p[j] / den;
          for (int d = 0; d < D; ++d) o[d] += w * __bfloat162float(vr[d]);
        }
      }
  char name[128];
  std::snprintf(name, sizeof name, "paged prefill, page %d, %dq/%dkv x %d, %d requests (rc %d)", page, Hq, Hkv, D, B, rc);
  report(name, want, got, 2e-2f);
  for (void* ptr : {(void*)dk, (void*)dv, (void*)dq, (void*)dout, (void*)dt, (void*)dr, (void*)dcq, (void*)dck}) CK(cudaFree(ptr));
}

}  // namespace

int main() {
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) {
    std::printf("no CUDA device: nothing checked\n");
    return 0;
  }
  int* status = device_zeros<int>(1);
  std::printf("GEMM family against CPU fp32 on the operands the kernels consumed\n");
  check_bf16(256, 384, 512, false, status);
  check_bf16(200, 136, 264, false, status);  // ragged M / N / K: partial tiles through the TMA fill
  check_bf16(512, 256, 320, true, status);
  check_fp8(256, 256, 512, false, status);
  check_fp8(192, 320, 272, true, status);
  check_fp8_block(256, 384, 512, status);
  check_fp8_block(136, 200, 256, status);
  check_int8(256, 256, 512, status);
  check_int8(100, 72, 144, status);
  std::printf("prefill attention over a paged pool against CPU fp32\n");
  check_paged_prefill(16, 8, 2, 128, {40, 1, 130, 64}, {40, 77, 300, 64}, status);
  check_paged_prefill(8, 4, 4, 64, {17, 256}, {200, 256}, status);
  check_paged_prefill(64, 6, 1, 128, {5, 90, 33}, {133, 90, 64}, status);
  int st = 0;
  CK(cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost));
  std::printf("  kernel status word: %d\n", st);
  if (st != 0) ++g_failures;
  std::printf("%s\n", g_failures ? "FAILED" : "all checks passed");
  return g_failures ? 1 : 0;
}
