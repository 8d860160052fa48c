// Paged decode attention with its scratch memory built into the library (see paged_decode_static.h for who needs
// this and for the limits).  The math is the split-KV kernel of paged_attention.cu, launched through the same host
// launcher; the only difference is where the split partials and counters live.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "launchers.h"
#include "paged_decode_static.h"

namespace {

constexpr long long kOPartFloats = (long long)ASTRAI_B200_NOALLOC_MAX_QELEMS * ASTRAI_B200_NOALLOC_MAX_SPLITS;
constexpr long long kMlPartFloats = (long long)ASTRAI_B200_NOALLOC_MAX_HEADS * ASTRAI_B200_NOALLOC_MAX_SPLITS * 2;
constexpr long long kCounterInts = ASTRAI_B200_NOALLOC_MAX_HEADS;
constexpr long long kOPartBytes = kOPartFloats * 4;
constexpr long long kMlPartBytes = kMlPartFloats * 4;  // a multiple of 256, so the counters stay aligned
constexpr long long kScratchBytes = kOPartBytes + kMlPartBytes + kCounterInts * 4;

// Layout: [ o_part fp32 | ml_part fp32 | counters int32 ].  Each GPU that loads the library holds one copy.
// In host code this name is only a handle for cudaGetSymbolAddress; it is not a pointer a kernel could use.
static __device__ __align__(256) unsigned char g_decode_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

thread_local char t_error[256] = "";

int fail(int code, const char* what) {
  snprintf(t_error, sizeof(t_error), "astrai_b200_paged_decode_noalloc: %s", what);
  return code;
}

int fail(int code, const char* what, long long a, long long b) {
  snprintf(t_error, sizeof(t_error), "astrai_b200_paged_decode_noalloc: %s (%lld, limit %lld)", what, a, b);
  return code;
}

// Device address of the scratch array on the current device; resolved once per device.
unsigned char* scratch_for_current_device(int* err) {
  int dev = -1;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *err = fail(-10, "cannot identify the current device", dev, kMaxDevices);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    rc = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (rc != cudaSuccess || p == nullptr) {
      snprintf(t_error, sizeof(t_error), "astrai_b200_paged_decode_noalloc: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(rc));
      *err = -11;
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int astrai_b200_paged_decode_noalloc(const void* q, const void* k_buf, const void* v_buf,
                                                const int* req_to_token, const int* req_pool_indices,
                                                const long long* seq_lens, void* out, int batch, int n_q_heads,
                                                int n_kv_heads, int head_dim, int max_ctx, long long n_slots,
                                                long long max_len, float scale, void* stream) {
  t_error[0] = 0;
  if (batch == 0) return 0;
  if (!q || !k_buf || !v_buf || !req_to_token || !req_pool_indices || !seq_lens || !out)
    return fail(-1, "null pointer argument");
  if (batch < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_ctx <= 0 || n_slots <= 0)
    return fail(-2, "non-positive size");
  if (head_dim != 32 && head_dim != 64 && head_dim != 128 && head_dim != 256)
    return fail(-3, "head_dim must be 32, 64, 128 or 256", head_dim, 256);
  const int group = n_q_heads % n_kv_heads == 0 ? n_q_heads / n_kv_heads : 0;
  if (group < 1 || group > 8) return fail(-4, "query heads per kv head must be between 1 and 8", group, 8);
  const long long q_elems = (long long)batch * n_q_heads * head_dim;
  if (q_elems > ASTRAI_B200_NOALLOC_MAX_QELEMS)
    return fail(-5, "batch * n_q_heads * head_dim exceeds the built-in scratch", q_elems, ASTRAI_B200_NOALLOC_MAX_QELEMS);
  if ((long long)batch * n_q_heads > ASTRAI_B200_NOALLOC_MAX_HEADS)
    return fail(-6, "batch * n_q_heads exceeds the built-in scratch", (long long)batch * n_q_heads,
                ASTRAI_B200_NOALLOC_MAX_HEADS);

  int err = 0;
  unsigned char* base = scratch_for_current_device(&err);
  if (base == nullptr) return err;
  float* o_part = reinterpret_cast<float*>(base);
  float* ml_part = reinterpret_cast<float*>(base + kOPartBytes);
  int* counters = reinterpret_cast<int*>(base + kOPartBytes + kMlPartBytes);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The counters must be zero when the kernel starts; an earlier call that was cut short could have left some set.
  cudaError_t rc = cudaMemsetAsync(counters, 0, sizeof(int) * (size_t)batch * n_kv_heads, st);
  if (rc != cudaSuccess) {
    snprintf(t_error, sizeof(t_error), "astrai_b200_paged_decode_noalloc: clearing counters failed: %s",
             cudaGetErrorString(rc));
    return -12;
  }
  const int splits = ab::paged_decode_splits(batch, n_kv_heads, max_len < 1 ? 1 : max_len, ASTRAI_B200_NOALLOC_MAX_SPLITS);
  const int lrc = ab::paged_decode(q, k_buf, v_buf, req_to_token, req_pool_indices, seq_lens, o_part, ml_part, counters,
                                   out, batch, n_q_heads, n_kv_heads, head_dim, max_ctx, n_slots, scale, splits,
                                   ASTRAI_B200_NOALLOC_MAX_SPLITS, /*table_rows: not known to a raw-pointer caller*/ 0, st);
  if (lrc != 0) return fail(-13, "kernel launch was rejected", lrc, 0);
  return 0;
}

extern "C" const char* astrai_b200_noalloc_error(void) { return t_error; }
