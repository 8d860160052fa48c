// Issue-rate probe for tcgen05.mma: one lane issues a long run of M=128 x N x K=16 bf16 MMAs on fixed (zeroed) shared
// memory tiles and the kernel reports SM clocks per instruction.  It answers two design questions for the kernels in
// this library: what the tensor core sustains for a given N, and how few scalar instructions the issuing lane may
// spend per MMA before it - not the tensor core - becomes the limit (`lean` = one 32-bit add per descriptor,
// otherwise the descriptor is rebuilt from the address for every instruction).
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"
#include "tcgen05.cuh"

namespace ab {
namespace {

using namespace tc;

template <int N>
__global__ void __launch_bounds__(128, 1) mma_issue_kernel(int reps, int lean, long long* __restrict__ out) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t holder;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 96 * 1024 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem_raw + (base - smem_u32(smem_raw)))[i] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = holder;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = idesc_bf16(128, N, false, false);
    const uint32_t a_smem = base, b_smem = base + 32 * 1024;
    const uint32_t a_lo = desc_lo(a_smem, true, 0), b_lo = desc_lo(b_smem, true, 0);
    const long long t0 = clock64();
#pragma unroll 1
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (lean) {
          tc_mma_lo(tmem, a_lo + 2 * k, b_lo + 2 * k, idesc, 1u);
        } else {
          tc_mma(tmem, smem_desc_sw128(a_smem + (r & 1) * 0, true, 0) + 2 * k, smem_desc_sw128(b_smem + (r & 1) * 0, true, 0) + 2 * k,
                 idesc, 1u);
        }
      }
    }
    tc_commit(smem_u32(&bar));
    volatile int never = 0;
    (void)mbar_wait(smem_u32(&bar), 0, &never);  // bounded
    const long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

template <int N>
int run(int reps, int lean, long long* out, cudaStream_t st) {
  constexpr int SMEM = 100 * 1024;
  if (cudaFuncSetAttribute(mma_issue_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -4;
  mma_issue_kernel<N><<<148, 128, SMEM, st>>>(reps, lean, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int mma_issue_bench(int n, int reps, bool lean, long long* out_cycles, cudaStream_t st) {
  switch (n) {
    case 64: return run<64>(reps, lean ? 1 : 0, out_cycles, st);
    case 128: return run<128>(reps, lean ? 1 : 0, out_cycles, st);
    case 256: return run<256>(reps, lean ? 1 : 0, out_cycles, st);
  }
  return -3;
}

}  // namespace ab
