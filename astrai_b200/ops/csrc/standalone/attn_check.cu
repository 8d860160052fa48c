// Torch-free check and timing of the attention kernels: links flash_fwd.cu and paged_attention.cu only, allocates with
// cudaMalloc, compares with a plain CPU fp32 attention, then times two serving-sized cases with CUDA events.
//   build:  python -m astrai_b200.ops.build --standalone      (writes astrai_b200/ops/build/attn_check)
//   run  :  astrai_b200/ops/build/attn_check                   (exit code 0 = every case within tolerance)
// Counterpart of the reference's torch-free test binaries with a CPU reference attention
// (csrc/tests/attn_test.cu:108-300, csrc/tests/attn_paged_test.cu:39-86, csrc/tests/test_utils.cuh:143-187).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
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

std::mt19937 g_rng(1234);

std::vector<__nv_bfloat16> random_bf16(size_t n, float scale = 1.f) {
  std::normal_distribution<float> d(0.f, scale);
  std::vector<__nv_bfloat16> v(n);
  for (auto& x : v) x = __float2bfloat16(d(g_rng));
  return v;
}

template <typename T>
T* to_device(const std::vector<T>& h) {
  T* d = nullptr;
  CK(cudaMalloc(&d, h.size() * sizeof(T)));
  CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}

// out[q, h, :] = softmax(scale * q . k^T + mask) v for one sequence; q [Sq, Hq, D], k / v [Sk, Hkv, D]; causal is
// lower-right aligned (query i sees keys <= i + Sk - Sq).
void cpu_attention(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, float* out, int Sq, int Sk, int Hq,
                   int Hkv, int D, float scale, bool causal) {
  const int G = Hq / Hkv;
  std::vector<float> p(Sk);
  for (int i = 0; i < Sq; ++i)
    for (int h = 0; h < Hq; ++h) {
      const int kvh = h / G, limit = causal ? std::min(Sk, i + Sk - Sq + 1) : Sk;
      float mx = -INFINITY;
      for (int j = 0; j < limit; ++j) {
        float s = 0.f;
        for (int d = 0; d < D; ++d)
          s += __bfloat162float(q[((size_t)i * Hq + h) * D + d]) * __bfloat162float(k[((size_t)j * Hkv + kvh) * D + d]);
        p[j] = s * scale;
        mx = std::max(mx, p[j]);
      }
      float l = 0.f;
      for (int j = 0; j < limit; ++j) l += (p[j] = std::exp(p[j] - mx));
      for (int d = 0; d < D; ++d) {
        float acc = 0.f;
        for (int j = 0; j < limit; ++j) acc += p[j] * __bfloat162float(v[((size_t)j * Hkv + kvh) * D + d]);
        out[((size_t)i * Hq + h) * D + d] = limit > 0 ? acc / l : 0.f;
      }
    }
}

float max_err(const std::vector<__nv_bfloat16>& got, const std::vector<float>& want) {
  float e = 0.f;
  for (size_t i = 0; i < want.size(); ++i) e = std::max(e, std::fabs(__bfloat162float(got[i]) - want[i]));
  return e;
}

int g_failures = 0;
void report(const char* what, float err, float tol) {
  std::printf("  %-58s max |err| %.4f  %s\n", what, err, err <= tol ? "ok" : "FAIL");
  if (!(err <= tol)) ++g_failures;
}

void check_flash(int B, int S, int Hq, int Hkv, int D, bool causal, int* status) {
  const size_t nq = (size_t)B * S * Hq * D, nk = (size_t)B * S * Hkv * D;
  auto q = random_bf16(nq), k = random_bf16(nk), v = random_bf16(nk);
  __nv_bfloat16 *dq = to_device(q), *dk = to_device(k), *dv = to_device(v), *dout = nullptr;
  float* dlse = nullptr;
  CK(cudaMalloc(&dout, nq * 2));
  CK(cudaMalloc(&dlse, (size_t)B * S * Hq * 4));
  const float scale = 1.f / std::sqrt((float)D);
  const int rc = ab::flash_fwd(dq, dk, dv, dout, dlse, nullptr, nullptr, B, S, S, S, (long long)B * S, (long long)B * S, Hq, Hkv, D,
                               (long long)Hq * D, (long long)Hkv * D, (long long)Hkv * D, (long long)Hq * D, scale, causal, status, 0);
  CK(cudaDeviceSynchronize());
  std::vector<__nv_bfloat16> got(nq);
  CK(cudaMemcpy(got.data(), dout, nq * 2, cudaMemcpyDeviceToHost));
  std::vector<float> want(nq);
  for (int b = 0; b < B; ++b)
    cpu_attention(q.data() + (size_t)b * S * Hq * D, k.data() + (size_t)b * S * Hkv * D, v.data() + (size_t)b * S * Hkv * D,
                  want.data() + (size_t)b * S * Hq * D, S, S, Hq, Hkv, D, scale, causal);
  char name[128];
  std::snprintf(name, sizeof(name), "flash_fwd B%d S%d %dq/%dkv D%d %s (rc %d)", B, S, Hq, Hkv, D, causal ? "causal" : "full", rc);
  report(name, rc == 0 ? max_err(got, want) : 1e9f, 0.03f);
  cudaFree(dq), cudaFree(dk), cudaFree(dv), cudaFree(dout), cudaFree(dlse);
}

struct DecodeCase {
  int B, Hq, Hkv, D, max_ctx;
  std::vector<long long> lens;
};

void check_decode(const DecodeCase& c, int* status) {
  const int B = c.B, max_splits = 8;
  long long total = 0;
  for (auto l : c.lens) total += l;
  const long long n_slots = total + 64;
  auto kbuf = random_bf16((size_t)n_slots * c.Hkv * c.D), vbuf = random_bf16((size_t)n_slots * c.Hkv * c.D);
  auto q = random_bf16((size_t)B * c.Hq * c.D);
  // every token of every request lives in a random distinct slot
  std::vector<int> slots(n_slots);
  for (long long i = 0; i < n_slots; ++i) slots[i] = (int)i;
  std::shuffle(slots.begin(), slots.end(), g_rng);
  std::vector<int> table((size_t)B * c.max_ctx, -1), rows(B);
  long long cur = 0;
  for (int b = 0; b < B; ++b) {
    rows[b] = b;
    for (long long t = 0; t < c.lens[b]; ++t) table[(size_t)b * c.max_ctx + t] = slots[cur++];
  }
  __nv_bfloat16 *dq = to_device(q), *dk = to_device(kbuf), *dv = to_device(vbuf), *dout = nullptr;
  int *dtable = to_device(table), *drows = to_device(rows), *dcnt = nullptr;
  long long* dlens = to_device(c.lens);
  float *dop = nullptr, *dml = nullptr;
  CK(cudaMalloc(&dout, q.size() * 2));
  CK(cudaMalloc(&dop, (size_t)B * c.Hq * max_splits * c.D * 4));
  CK(cudaMalloc(&dml, (size_t)B * c.Hq * max_splits * 2 * 4));
  CK(cudaMalloc(&dcnt, (size_t)B * c.Hkv * 4));
  CK(cudaMemset(dcnt, 0, (size_t)B * c.Hkv * 4));
  const float scale = 1.f / std::sqrt((float)c.D);
  const long long longest = *std::max_element(c.lens.begin(), c.lens.end());
  const int splits = ab::paged_decode_splits(B, c.Hkv, longest, max_splits);
  int rc = 0;
  for (int rep = 0; rep < 2 && rc == 0; ++rep)  // twice: the counters must reset themselves
    rc = ab::paged_decode(dq, dk, dv, dtable, drows, dlens, dop, dml, dcnt, dout, B, c.Hq, c.Hkv, c.D, c.max_ctx, n_slots, scale, splits,
                          max_splits, B, 0);
  CK(cudaDeviceSynchronize());
  std::vector<__nv_bfloat16> got(q.size());
  CK(cudaMemcpy(got.data(), dout, q.size() * 2, cudaMemcpyDeviceToHost));
  std::vector<float> want(q.size());
  for (int b = 0; b < B; ++b) {
    const long long L = c.lens[b];
    std::vector<__nv_bfloat16> ks((size_t)L * c.Hkv * c.D), vs((size_t)L * c.Hkv * c.D);
    for (long long t = 0; t < L; ++t) {
      const size_t slot = (size_t)table[(size_t)b * c.max_ctx + t];
      std::copy_n(kbuf.begin() + slot * c.Hkv * c.D, (size_t)c.Hkv * c.D, ks.begin() + (size_t)t * c.Hkv * c.D);
      std::copy_n(vbuf.begin() + slot * c.Hkv * c.D, (size_t)c.Hkv * c.D, vs.begin() + (size_t)t * c.Hkv * c.D);
    }
    cpu_attention(q.data() + (size_t)b * c.Hq * c.D, ks.data(), vs.data(), want.data() + (size_t)b * c.Hq * c.D, 1, (int)L, c.Hq, c.Hkv,
                  c.D, scale, false);
  }
  char name[128];
  std::snprintf(name, sizeof(name), "paged_decode B%d %dq/%dkv D%d splits %d (rc %d)", B, c.Hq, c.Hkv, c.D, splits, rc);
  report(name, rc == 0 ? max_err(got, want) : 1e9f, 0.03f);
  cudaFree(dq), cudaFree(dk), cudaFree(dv), cudaFree(dout), cudaFree(dtable), cudaFree(drows), cudaFree(dcnt), cudaFree(dlens);
  cudaFree(dop), cudaFree(dml);
}

float time_ms(int reps, const std::function<void()>& fn) {
  for (int i = 0; i < 3; ++i) fn();
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e0));
  for (int i = 0; i < reps; ++i) fn();
  CK(cudaEventRecord(e1));
  CK(cudaEventSynchronize(e1));
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, e0, e1));
  return ms / reps;
}
}  // namespace

int main() {
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count == 0) {
    std::printf("no CUDA device: nothing checked\n");
    return 0;
  }
  int* status = nullptr;
  CK(cudaMalloc(&status, 4));
  CK(cudaMemset(status, 0, 4));
  std::printf("correctness against CPU fp32 attention\n");
  check_flash(2, 300, 4, 2, 64, true, status);
  check_flash(1, 257, 8, 2, 128, true, status);
  check_flash(2, 128, 4, 4, 128, false, status);
  check_flash(1, 77, 6, 1, 64, false, status);
  check_decode({3, 8, 2, 128, 512, {1, 77, 500}}, status);
  check_decode({4, 24, 4, 64, 1024, {1000, 16, 333, 129}}, status);
  check_decode({2, 4, 4, 256, 256, {200, 5}}, status);
  check_decode({5, 5, 1, 32, 128, {128, 1, 2, 64, 99}}, status);
  int st = 0;
  CK(cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost));
  std::printf("  kernel status word: %d\n", st);
  if (st != 0) ++g_failures;

  std::printf("timing (CUDA events, 3 warm-ups, mean of 20)\n");
  {
    const int B = 4, S = 2048, Hq = 16, Hkv = 4, D = 128;
    const size_t nq = (size_t)B * S * Hq * D, nk = (size_t)B * S * Hkv * D;
    auto q = random_bf16(nq), k = random_bf16(nk), v = random_bf16(nk);
    __nv_bfloat16 *dq = to_device(q), *dk = to_device(k), *dv = to_device(v), *dout = nullptr;
    float* dlse = nullptr;
    CK(cudaMalloc(&dout, nq * 2));
    CK(cudaMalloc(&dlse, (size_t)B * S * Hq * 4));
    const float ms = time_ms(20, [&] {
      ab::flash_fwd(dq, dk, dv, dout, dlse, nullptr, nullptr, B, S, S, S, (long long)B * S, (long long)B * S, Hq, Hkv, D, (long long)Hq * D,
                    (long long)Hkv * D, (long long)Hkv * D, (long long)Hq * D, 1.f / std::sqrt((float)D), true, status, 0);
    });
    const double flop = 4.0 * B * (double)S * S * Hq * D / 2;
    std::printf("  flash_fwd B4 S2048 16q/4kv D128 causal: %.1f us, %.0f TFLOP/s\n", ms * 1e3, flop / ms / 1e9);
  }
  std::printf("%s\n", g_failures ? "FAILED" : "all checks passed");
  return g_failures ? 1 : 0;
}
