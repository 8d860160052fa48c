// Host-side creation and caching of 2-D bf16 tensor maps (128-byte swizzle) for the tcgen05 kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <tuple>

namespace ab {
namespace tmah {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row stride ld elements.
inline thread_local int g_last_map_error = 0;

inline bool make_map(CUtensorMap* out, const void* ptr, long long inner, long long outer, long long ld, int box_inner,
              int box_outer) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    g_last_map_error = -1;
    return false;
  }
  // The driver entry point needs a current context; a fresh thread (autograd worker) has none until its first
  // runtime call, so make one here (only on a cache miss).
  // Once per thread is enough, and it must not run while the stream is being captured into a CUDA graph
  // (the warm-up pass before a capture has already bound the context).
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUresult res = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_map_error = (int)res;
  return res == CUDA_SUCCESS;
}

struct MapCache {
  using Key = std::tuple<const void*, long long, long long, long long, int, int>;
  std::map<Key, CUtensorMap> maps;
  std::mutex mu;
  bool get(CUtensorMap* out, const void* ptr, long long inner, long long outer, long long ld, int bi, int bo) {
    Key k{ptr, inner, outer, ld, bi, bo};
    std::lock_guard<std::mutex> g(mu);
    auto it = maps.find(k);
    if (it == maps.end()) {
      CUtensorMap m;
      if (!make_map(&m, ptr, inner, outer, ld, bi, bo)) return false;
      if (maps.size() > 4096) maps.clear();
      it = maps.emplace(k, m).first;
    }
    *out = it->second;
    return true;
  }
};
inline MapCache& cache() {
  static MapCache c;
  return c;
}


}  // namespace tmah
}  // namespace ab
