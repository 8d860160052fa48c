// Flash attention backward on tcgen05 (sm_100a), as two deterministic kernels (no atomics) plus a row-dot pre-pass:
//
//   flash_delta      : delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]
//   flash_bwd_dkdv   : one CTA per (128-key tile, kv head, sequence).  K and V stay resident in shared memory; the CTA
//                      walks over the query heads of its GQA group and over 64-query sub-tiles:
//                        S^T = K Q^T, dP^T = V dO^T        (tcgen05, M=128 keys, N=64 queries, double-buffered in TMEM)
//                        P^T = exp2(S^T c - lse), dS^T = P^T (dP^T - delta)     (one thread per key row; two warp groups alternate sub-tiles)
//                        dV += P^T dO, dK += dS^T Q        (tcgen05, accumulators live in TMEM for the whole CTA)
//   flash_bwd_dq     : one CTA per (128-query tile, query head, sequence).  Q and dO stay resident; the CTA walks over
//                      64-key sub-tiles: S = Q K^T, dP = dO V^T, dS = P (dP - delta), dQ += dS K.  The softmax scale is applied
//                      to dK and dQ once, when the accumulators are written out.
// P^T / dS^T / dS are written by the row threads into shared memory in the 128-byte-swizzled K-major layout and consumed
// as the A operand of the accumulating MMAs; dO, Q and K are consumed as MN-major B operands straight from the tiles TMA
// delivered (no transposes are materialised).  Recomputing S and dP in the second kernel costs two extra GEMMs per tile
// pair and buys a backward pass without fp32 atomics, with a fixed summation order.
// Layouts, masking and GQA conventions are those of flash_fwd.cu.  Replaces the backward of
// F.scaled_dot_product_attention in the reference's training path (astrai/extension/backend/attention.py:453-468).
// All mbarrier waits are bounded; on expiry the CTA records a code in `status` and leaves through the common exit.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flash_cp.cuh"
#include "launchers.h"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace ab {
namespace {

using namespace tc;
using namespace tmah;
using namespace cpx;

constexpr int BWD_THREADS = 320, SUB = 64, QDO_STAGES = 4, KV_STAGES_B = 6;  // warp 0 TMA, warp 1 MMA, warps 2..9 rows (two per TMEM quarter)
constexpr int DQ_GROUPS = 3, V_STAGES_B = 4, DQ_THREADS = 64 + DQ_GROUPS * 128;  // dQ kernel: three row-warp groups, V released earlier than K
constexpr int BLK128 = 128 * 128;  // [128 rows x 64 cols] swizzled block
constexpr int BLK64 = 64 * 128;    // [64 rows x 64 cols] swizzled block
constexpr float LOG2E = 1.4426950408889634f;
// mbarrier slots.  dK/dV kernel: kv_full | qdo_full[S] | qdo_empty[S] | s_full[2] | pds_full[2] | pds_empty[2] | done
enum : int { A_QF = 1, A_QE = 1 + QDO_STAGES, A_SF = 1 + 2 * QDO_STAGES, A_PF = 3 + 2 * QDO_STAGES, A_PE = 5 + 2 * QDO_STAGES,
             A_DONE = 7 + 2 * QDO_STAGES, A_NBAR = 8 + 2 * QDO_STAGES };
// dQ kernel: qdo_full | k_full[S] | k_empty[S] | v_full[S] | v_empty[S] | s_full[G] | ds_full[G] | ds_empty[G] | done
enum : int { B_KF = 1, B_KE = 1 + KV_STAGES_B, B_VF = 1 + 2 * KV_STAGES_B, B_VE = 1 + 3 * KV_STAGES_B, B_SF = 1 + 4 * KV_STAGES_B,
             B_DF = B_SF + DQ_GROUPS, B_DE = B_DF + DQ_GROUPS, B_DONE = B_DE + DQ_GROUPS, B_NBAR = B_DONE + 1 };
enum : int { ERR_BWD_PRODUCER = 41, ERR_BWD_MMA = 42, ERR_BWD_ROWS = 43 };

struct SeqInfoB {
  int q_start, q_len, k_start, k_len;
};
__device__ __forceinline__ SeqInfoB seq_info_b(const int* cu_q, const int* cu_k, int b, int sq, int sk) {
  SeqInfoB s;
  s.q_start = cu_q ? cu_q[b] : b * sq;
  s.q_len = cu_q ? cu_q[b + 1] - cu_q[b] : sq;
  s.k_start = cu_k ? cu_k[b] : b * sk;
  s.k_len = cu_k ? cu_k[b + 1] - cu_k[b] : sk;
  return s;
}

// ------------------------------------------------------------------------------------------------ delta pre-pass
template <int D>
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                   const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                                   long long total_q, int Hq, long long do_stride, long long o_stride) {
  // D/8 lanes carry 16 bytes each of one (token, head) row: a warp covers 32 / (D/8) rows at a time
  constexpr int LPR = D / 8, RPW = 32 / LPR;  // lanes per row, rows per warp
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long r = w * RPW + lane / LPR;
  const int sub = lane % LPR;
  const bool live = r < total_q * Hq;
  const long long t = live ? r / Hq : 0;
  const int h = live ? (int)(r % Hq) : 0;
  float acc = 0.f;
  if (live) {
    const uint4 a = *reinterpret_cast<const uint4*>(dO + t * do_stride + (long long)h * D + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(O + t * o_stride + (long long)h * D + sub * 8);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (live && sub == 0) {
    delta[(long long)h * total_q + t] = acc;
    lse2[(long long)h * total_q + t] = lse[(long long)h * total_q + t] * LOG2E;
  }
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Write 32-column chunks [c_begin, c_end) of one accumulator row (fp32 in TMEM at taddr) times `mult` as bf16 to `dst`.
__device__ __forceinline__ void store_acc_row(uint32_t taddr, __nv_bfloat16* dst, bool live, bool have, int c_begin,
                                              int c_end, float mult) {
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t o[32];
    if (have) {
      tc_ld32(taddr + c * 32, o);
      tc_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0u;
    }
    if (live) {
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        uint4 pkd;
        uint32_t* pw = reinterpret_cast<uint32_t*>(&pkd);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          pw[q] = pack2(__uint_as_float(o[8 * v4 + 2 * q]) * mult, __uint_as_float(o[8 * v4 + 2 * q + 1]) * mult);
        reinterpret_cast<uint4*>(dst + c * 32)[v4] = pkd;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ dK / dV
template <int D>
struct DkvCfg {
  static constexpr int NB = D / 64;
  static constexpr int KV_BYTES = 128 * D * 2;   // resident K or V tile
  static constexpr int QS_BYTES = SUB * D * 2;   // one 64-row Q or dO stage
  static constexpr int ROW_BYTES = 2 * SUB * 4;   // lse (log2 units) and delta of one sub-tile's queries
  static constexpr int SMEM = 2 * KV_BYTES + 2 * QDO_STAGES * QS_BYTES + 1024 + 256 + QDO_STAGES * ROW_BYTES;
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                      const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const float* __restrict__ lse2g, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK,
                      __nv_bfloat16* __restrict__ dV, const int* __restrict__ cu_q, const int* __restrict__ cu_k, int sq,
                      int sk, int Hq, int Hkv, long long dk_row_stride, long long total_q, float scale, int causal,
                      int* __restrict__ status, const CpAttn cp) {
  using C = DkvCfg<D>;
  // grid = (kv heads x sequences, key tiles): blocks are dispatched in linear order, so every key tile 0 (the one
  // with the most query tiles under a causal mask) starts before any lighter tile - longest work first.
  const int kvh = (int)blockIdx.x % Hkv;
  const int bseq = (int)blockIdx.x / Hkv;
  SeqInfoB si = seq_info_b(cu_q, cu_k, bseq, sq, sk);
  if (cp.world > 1) si.k_len = cp.k_vis;
  const int k0 = (int)blockIdx.y * 128;
  if (k0 >= si.k_len) return;
  const int G = Hq / Hkv;
  // Query rows come in two ranges with their own causal offset: [0, split) at off_a (context parallel only) and
  // [split, q_len) at off_b.  Of each range only the 64-row sub-tiles that can see this key tile are visited.
  const int split = cp.world > 1 ? cp.chunk : 0;
  const int off_a = cp.rank * cp.chunk, off_b = si.k_len - si.q_len;
  int lo1 = 0, lo2 = split;
  if (causal) {
    lo1 = min(split, max(0, k0 - off_a) / SUB * SUB);
    lo2 = max(split, max(0, k0 - off_b) / SUB * SUB);
  }
  const int n1 = (split - lo1) / SUB;
  const int n_sub = n1 + max(0, (si.q_len - lo2 + SUB - 1) / SUB);
  const int n_it = n_sub * G;
  auto sub_start = [&](int idx) { return idx < n1 ? lo1 + idx * SUB : lo2 + (idx - n1) * SUB; };

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t k_smem = base, v_smem = base + C::KV_BYTES;
  const uint32_t q_smem = v_smem + C::KV_BYTES;                    // QDO_STAGES stages
  const uint32_t do_smem = q_smem + QDO_STAGES * C::QS_BYTES;      // QDO_STAGES stages
  uint8_t* tail = aligned + (do_smem + QDO_STAGES * C::QS_BYTES - base);  // barriers, TMEM address, statistics ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + A_NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  // per Q/dO stage: 64 lse values then 64 delta values of the sub-tile's queries, staged by the producer warp so that
  // the row threads never wait on global memory inside the loop
  float* row_stats = reinterpret_cast<float*>(tail + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < A_NBAR; ++i)
      mbar_init(BAR(i), (i == A_PF || i == A_PF + 1) ? 4 : (i >= A_QF && i < A_QF + QDO_STAGES) ? 2 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_dv = tmem_base + 256, tmem_dk = tmem_base + 384;

  if (warp == 0) {
    if (n_it > 0) {
      if (lane == 0) {
        mbar_expect_tx(BAR(0), 2 * C::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < C::NB; ++kb) {
          tma_load_2d(k_smem + kb * BLK128, &map_k, BAR(0), kvh * D + kb * 64, si.k_start + k0);
          tma_load_2d(v_smem + kb * BLK128, &map_v, BAR(0), kvh * D + kb * 64, si.k_start + k0);
        }
      }
      // Lane l carries lse and delta of queries 2l, 2l+1 of a sub-tile; the values of sub-tile it + 1 are requested
      // before the wait for its stage, so their latency is hidden behind the wait.  Queries past the sequence end get
      // lse = +inf (probability 0) and delta = 0.
      auto fetch = [&](int it, float2& lv, float2& dv) {
        const int h = kvh * G + it / n_sub, q = sub_start(it % n_sub) + 2 * lane;
        const long long o = (long long)h * total_q + si.q_start + q;
        lv.x = q < si.q_len ? __ldg(lse2g + o) : INFINITY;
        lv.y = q + 1 < si.q_len ? __ldg(lse2g + o + 1) : INFINITY;
        dv.x = q < si.q_len ? __ldg(delta + o) : 0.f;
        dv.y = q + 1 < si.q_len ? __ldg(delta + o + 1) : 0.f;
      };
      float2 lv, dv;
      fetch(0, lv, dv);
      bool ok = true;
      for (int it = 0; it < n_it; ++it) {
        const int st = it % QDO_STAGES;
        const uint32_t ph = ((it / QDO_STAGES) & 1) ^ 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(BAR(A_QE + st), ph, abort_flag));
        if (!ok) break;
        if (lane == 0) {
          const int h = kvh * G + it / n_sub, qs = sub_start(it % n_sub);
          mbar_expect_tx(BAR(A_QF + st), 2 * C::QS_BYTES);
#pragma unroll
          for (int kb = 0; kb < C::NB; ++kb) {
            tma_load_2d(q_smem + st * C::QS_BYTES + kb * BLK64, &map_q, BAR(A_QF + st), h * D + kb * 64, si.q_start + qs);
            tma_load_2d(do_smem + st * C::QS_BYTES + kb * BLK64, &map_do, BAR(A_QF + st), h * D + kb * 64, si.q_start + qs);
          }
        }
        float* rs = row_stats + st * (2 * SUB);
        reinterpret_cast<float2*>(rs)[lane] = lv;
        reinterpret_cast<float2*>(rs + SUB)[lane] = dv;
        if (it + 1 < n_it) fetch(it + 1, lv, dv);
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(A_QF + st));  // second arrival of the stage: the statistics are in place
      }
      if (!ok && lane == 0) {
        atomicMax(status, ERR_BWD_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_sc = idesc_bf16(128, SUB, false, false);
      constexpr uint32_t idesc_acc = idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(BAR(0), 0, abort_flag);
      const uint32_t k_lo = desc_lo(k_smem, true, 0), v_lo = desc_lo(v_smem, true, 0);
      const uint32_t q_lo0 = desc_lo(q_smem, true, 0), do_lo0 = desc_lo(do_smem, true, 0);
      const uint32_t qmn_lo0 = desc_lo(q_smem, false, BLK64), domn_lo0 = desc_lo(do_smem, false, BLK64);
      auto issue_scores = [&](int it) -> bool {
        const int st = it % QDO_STAGES, buf = it & 1;
        if (!mbar_wait(BAR(A_QF + st), (it / QDO_STAGES) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q_lo = q_lo0 + st * (C::QS_BYTES >> 4), do_lo = do_lo0 + st * (C::QS_BYTES >> 4);
        const uint32_t d_s = tmem_base + buf * SUB, d_dp = tmem_base + 128 + buf * SUB;
#pragma unroll
        for (int kb = 0; kb < C::NB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tc_mma_lo(d_s, k_lo + kb * (BLK128 >> 4) + 2 * k, q_lo + kb * (BLK64 >> 4) + 2 * k, idesc_sc, (kb | k) ? 1u : 0u);
            tc_mma_lo(d_dp, v_lo + kb * (BLK128 >> 4) + 2 * k, do_lo + kb * (BLK64 >> 4) + 2 * k, idesc_sc, (kb | k) ? 1u : 0u);
          }
        tc_commit(BAR(A_SF + buf));
        return true;
      };
      if (ok) ok = issue_scores(0);
      if (ok && n_it > 1) ok = issue_scores(1);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % QDO_STAGES;
        const int g = it & 1;
        if (!mbar_wait(BAR(A_PF + g), (it >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pt_t = tmem_base + g * SUB, dst_t = tmem_base + 128 + g * SUB;  // P^T / dS^T over the score buffers
        const uint32_t domn_lo = domn_lo0 + st * (C::QS_BYTES >> 4), qmn_lo = qmn_lo0 + st * (C::QS_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          tc_mma_ts(tmem_dv, pt_t + 8 * k, domn_lo + k * 128, idesc_acc, (it | k) ? 1u : 0u);
          tc_mma_ts(tmem_dk, dst_t + 8 * k, qmn_lo + k * 128, idesc_acc, (it | k) ? 1u : 0u);
        }
        tc_commit(BAR(A_QE + st));  // Q / dO stage free
        tc_commit(BAR(A_PE + g));  // this group's P^T / dS^T consumed
        if (it + 2 < n_it && !issue_scores(it + 2)) { ok = false; break; }
      }
      if (ok) tc_commit(BAR(A_DONE));  // every accumulating MMA has retired
      if (!ok) {
        atomicMax(status, ERR_BWD_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    // Two groups of four warps; group g takes the sub-tiles it = g, g+2, ... with its own TMEM score buffers and its own
    // P^T / dS^T tiles, so one group's tcgen05.ld / smem-store / barrier latencies overlap the other group's math.
    const int quarter = warp & 3, g = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;        // key row of this thread
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int kidx = k0 + row;
    const bool key_live = kidx < si.k_len;
    const float scale_log2 = scale * LOG2E;
    bool ok = true;
    for (int it = g; it < n_it; it += 2) {
      const int qs = sub_start(it % n_sub);
      const int off = qs < split ? off_a : off_b;
      const int qmin = causal ? kidx - off : -0x40000000;  // query q sees this key iff q >= kidx - off
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(A_SF + g), (it >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      // the stage's statistics were published with the second arrival on its full barrier (phase long complete here)
      const int st = it % QDO_STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(A_QF + st), (it / QDO_STAGES) & 1, abort_flag));
      if (!ok) break;
      const float* lp0 = row_stats + st * (2 * SUB);
      const float* dlp0 = lp0 + SUB;
      const bool need_mask = (k0 + 128 > si.k_len) || (causal && qs < k0 + 127 - off);
      uint32_t ppk[32], dpk[32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t s[32], dp[32];
        tc_ld32(t_lane + g * SUB + half * 32, s);
        tc_ld32(t_lane + 128 + g * SUB + half * 32, dp);
        tc_wait_ld();
        const int qc = qs + half * 32;
        const float* lp = lp0 + half * 32;
        const float* dlp = dlp0 + half * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float lv[4], dv[4];
          *reinterpret_cast<float4*>(lv) = *reinterpret_cast<const float4*>(lp + i);
          *reinterpret_cast<float4*>(dv) = *reinterpret_cast<const float4*>(dlp + i);
          float pv[4], dsv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pe = ex2(fmaf(__uint_as_float(s[i + e]), scale_log2, -lv[e]));
            if (need_mask && (!key_live || qc + i + e < qmin)) pe = 0.f;
            pv[e] = pe;
            dsv[e] = pe * (__uint_as_float(dp[i + e]) - dv[e]);
          }
          ppk[half * 16 + (i >> 1)] = pack2(pv[0], pv[1]);
          ppk[half * 16 + (i >> 1) + 1] = pack2(pv[2], pv[3]);
          dpk[half * 16 + (i >> 1)] = pack2(dsv[0], dsv[1]);
          dpk[half * 16 + (i >> 1) + 1] = pack2(dsv[2], dsv[3]);
        }
      }
      // P^T and dS^T go back into tensor memory, over the first 32 columns of this group's S^T and dP^T buffers (both are
      // in registers by now); the dV / dK MMAs read them as A operands, and the scores of sub-tile it + 2, issued after
      // those MMAs by the same thread, overwrite them in order.
      tc_st32(t_lane + g * SUB, ppk);
      tc_st32(t_lane + 128 + g * SUB, dpk);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(A_PF + g));
    }
    if (ok && n_it > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(A_DONE), 0, abort_flag));
      if (ok) tc_fence_after();
    }
    const int half = g;  // each group writes half of the accumulator columns
    if (ok) {
      constexpr int CH = D / 64;  // 32-column chunks per half
      __nv_bfloat16 *dv_row, *dk_row;
      if (cp.world > 1 && cp.stage[0] != nullptr) {
        // context parallel: the tile goes to the staging slot [this rank] of the rank that owns these keys
        const int ch = k0 / cp.chunk, owner = chunk_owner(ch, cp.world);
        const long long local_row = (ch >= cp.world ? cp.chunk : 0) + (kidx - ch * cp.chunk);
        const long long row_elems = (long long)Hkv * D, plane = (long long)cp.batch * 2 * cp.chunk * row_elems;
        __nv_bfloat16* slot = reinterpret_cast<__nv_bfloat16*>(cp.stage[owner]) + (long long)cp.rank * 2 * plane;
        dk_row = slot + ((long long)bseq * 2 * cp.chunk + local_row) * row_elems + (long long)kvh * D;
        dv_row = dk_row + plane;
      } else {
        const long long tok = (long long)si.k_start + kidx;
        dv_row = dV + tok * dk_row_stride + (long long)kvh * D;
        dk_row = dK + tok * dk_row_stride + (long long)kvh * D;
      }
      store_acc_row(t_lane + 256, dv_row, key_live, n_it > 0, half * CH, half * CH + CH, 1.f);
      store_acc_row(t_lane + 384, dk_row, key_live, n_it > 0, half * CH, half * CH + CH, scale);
      if (cp.world > 1 && cp.stage[0] != nullptr) __threadfence_system();
    } else if (lane == 0) {
      atomicMax(status, ERR_BWD_ROWS);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (cp.world > 1 && cp.stage[0] != nullptr && threadIdx.x == 0 && *abort_flag == 0) {
    // the last tile this rank owes an owner tells it that the slot is complete
    const int owner = chunk_owner(k0 / cp.chunk, cp.world);
    const int expected = (1 + (owner >= cp.rank ? 1 : 0)) * (cp.chunk / 128) * Hkv * cp.batch;
    const int done = atomicAdd(&cp.tile_counter[owner], 1);
    if (done == expected - 1) {
      cp.tile_counter[owner] = 0;
      __threadfence_system();
      comm::st_release_sys(flag_slot(cp.flags[owner], KIND_CP_DKV, cp.rank, cp.unit, cp.max_units), cp.epoch);
    }
  }
}

// Owner side of the context-parallel dK / dV scatter: sum the contributors' staging slots.  Local rows [0, c) (chunk
// `rank`) are seen by every rank, rows [c, 2c) (chunk 2W - 1 - rank) by the ranks 0..rank.
__global__ void cp_dkv_reduce_kernel(__nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, long long row_elems,
                                     const CpAttn cp, int* __restrict__ status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int src = 0; src < cp.world && ok; ++src)
      ok = comm::wait_flag(flag_slot(cp.flags[cp.rank], KIND_CP_DKV, src, cp.unit, cp.max_units), cp.epoch, cp.timeout_ns) ? 1 : 0;
    if (!ok) atomicMax(status, ERR_CP_REDUCE);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const long long vec_per_row = row_elems / 8, rows = (long long)cp.batch * 2 * cp.chunk;
  const long long plane_vec = rows * vec_per_row, total = 2 * plane_vec;
  const uint4* stage = reinterpret_cast<const uint4*>(cp.stage[cp.rank]);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const long long in_plane = v % plane_vec;
    const int local_row = (int)((in_plane / vec_per_row) % (2 * cp.chunk));
    const int n_src = local_row < cp.chunk ? cp.world : cp.rank + 1;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int src = 0; src < n_src; ++src) {
      const uint4 x = comm::ld_sys_u4(stage + (long long)src * total + v);
      const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(px[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 o;
    uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) po[i] = pack2(acc[2 * i], acc[2 * i + 1]);
    uint4* out = reinterpret_cast<uint4*>(v < plane_vec ? dk : dv);
    out[in_plane] = o;
  }
}

// ------------------------------------------------------------------------------------------------ dQ
template <int D>
struct DqCfg {
  static constexpr int NB = D / 64;
  static constexpr int Q_BYTES = 128 * D * 2;   // resident Q or dO tile
  static constexpr int KS_BYTES = SUB * D * 2;  // one 64-key K or V stage
  static constexpr int SMEM = 2 * Q_BYTES + (KV_STAGES_B + V_STAGES_B) * KS_BYTES + 1024 + 512;  // 35 barriers need more than 256 bytes
  static_assert(B_NBAR * 8 + 16 <= 512, "barrier area");
};

template <int D>
__global__ void __launch_bounds__(DQ_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const float* __restrict__ lse2g, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dQ,
                    const int* __restrict__ cu_q, const int* __restrict__ cu_k, int sq, int sk, int Hq, int Hkv,
                    long long dq_row_stride, long long total_q, float scale, int causal, int* __restrict__ status,
                    const CpAttn cp) {
  using C = DqCfg<D>;
  // grid = (query heads x sequences, query tiles), heaviest (last) causal tiles dispatched first
  const int h = (int)blockIdx.x % Hq;
  SeqInfoB si = seq_info_b(cu_q, cu_k, (int)blockIdx.x / Hq, sq, sk);
  if (cp.world > 1) si.k_len = cp.k_vis;
  const int n_q_tiles = (si.q_len + 127) / 128;
  const int qt = n_q_tiles - 1 - (int)blockIdx.y;
  if (qt < 0) return;
  const int kvh = h / (Hq / Hkv);
  const int q0 = qt * 128;
  const int off = (cp.world > 1 && q0 < cp.chunk) ? cp.rank * cp.chunk : si.k_len - si.q_len;
  int kv_end = si.k_len;
  if (causal) kv_end = min(si.k_len, q0 + 128 + off);
  if (kv_end < 0) kv_end = 0;
  const int n_it = (kv_end + SUB - 1) / SUB;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base, do_smem = base + C::Q_BYTES;
  const uint32_t k_smem = do_smem + C::Q_BYTES;                 // stages
  const uint32_t v_smem = k_smem + KV_STAGES_B * C::KS_BYTES;    // stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (v_smem + V_STAGES_B * C::KS_BYTES - base));
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + B_NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < B_NBAR; ++i) mbar_init(BAR(i), (i >= B_DF && i < B_DF + DQ_GROUPS) ? 4 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // columns: S of the three groups (3 x 64) | dP of the three groups (3 x 64) | dQ (128)
  const uint32_t tmem_dq = tmem_base + 2 * DQ_GROUPS * SUB;

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(BAR(0), 2 * C::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < C::NB; ++kb) {
        tma_load_2d(q_smem + kb * BLK128, &map_q, BAR(0), h * D + kb * 64, si.q_start + q0);
        tma_load_2d(do_smem + kb * BLK128, &map_do, BAR(0), h * D + kb * 64, si.q_start + q0);
      }
      bool ok = true;
      for (int j = 0; j < n_it && ok; ++j) {
        const int st = j % KV_STAGES_B, sv = j % V_STAGES_B;
        if (!mbar_wait(BAR(B_KE + st), ((j / KV_STAGES_B) & 1) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(BAR(B_KF + st), C::KS_BYTES);
#pragma unroll
        for (int kb = 0; kb < C::NB; ++kb)
          tma_load_2d(k_smem + st * C::KS_BYTES + kb * BLK64, &map_k, BAR(B_KF + st), kvh * D + kb * 64, si.k_start + j * SUB);
        if (!mbar_wait(BAR(B_VE + sv), ((j / V_STAGES_B) & 1) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(BAR(B_VF + sv), C::KS_BYTES);
#pragma unroll
        for (int kb = 0; kb < C::NB; ++kb)
          tma_load_2d(v_smem + sv * C::KS_BYTES + kb * BLK64, &map_v, BAR(B_VF + sv), kvh * D + kb * 64, si.k_start + j * SUB);
      }
      if (!ok) {
        atomicMax(status, ERR_BWD_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_sc = idesc_bf16(128, SUB, false, false);
      constexpr uint32_t idesc_acc = idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(BAR(0), 0, abort_flag);
      const uint32_t q_lo = desc_lo(q_smem, true, 0), do_lo = desc_lo(do_smem, true, 0);
      const uint32_t k_lo0 = desc_lo(k_smem, true, 0), v_lo0 = desc_lo(v_smem, true, 0);
      const uint32_t kmn_lo0 = desc_lo(k_smem, false, BLK64);
      auto issue_scores = [&](int j) -> bool {
        const int st = j % KV_STAGES_B, sv = j % V_STAGES_B, buf = j % DQ_GROUPS;
        if (!mbar_wait(BAR(B_KF + st), (j / KV_STAGES_B) & 1, abort_flag) || !mbar_wait(BAR(B_VF + sv), (j / V_STAGES_B) & 1, abort_flag))
          return false;
        tc_fence_after();
        const uint32_t k_lo = k_lo0 + st * (C::KS_BYTES >> 4), v_lo = v_lo0 + sv * (C::KS_BYTES >> 4);
        const uint32_t d_s = tmem_base + buf * SUB, d_dp = tmem_base + (DQ_GROUPS + buf) * SUB;
#pragma unroll
        for (int kb = 0; kb < C::NB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tc_mma_lo(d_s, q_lo + kb * (BLK128 >> 4) + 2 * k, k_lo + kb * (BLK64 >> 4) + 2 * k, idesc_sc, (kb | k) ? 1u : 0u);
            tc_mma_lo(d_dp, do_lo + kb * (BLK128 >> 4) + 2 * k, v_lo + kb * (BLK64 >> 4) + 2 * k, idesc_sc, (kb | k) ? 1u : 0u);
          }
        tc_commit(BAR(B_VE + sv));  // V stage free
        tc_commit(BAR(B_SF + buf));
        return true;
      };
      for (int j = 0; j < DQ_GROUPS && j < n_it && ok; ++j) ok = issue_scores(j);
      for (int j = 0; j < n_it && ok; ++j) {
        const int st = j % KV_STAGES_B;
        const int g = j % DQ_GROUPS;
        if (!mbar_wait(BAR(B_DF + g), (j / DQ_GROUPS) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ds_t = tmem_base + (DQ_GROUPS + g) * SUB, kmn_lo = kmn_lo0 + st * (C::KS_BYTES >> 4);  // dS over dP
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_ts(tmem_dq, ds_t + 8 * k, kmn_lo + k * 128, idesc_acc, (j | k) ? 1u : 0u);
        tc_commit(BAR(B_KE + st));  // K stage free
        tc_commit(BAR(B_DE + g));  // this group's dS consumed
        if (j + DQ_GROUPS < n_it && !issue_scores(j + DQ_GROUPS)) { ok = false; break; }
      }
      if (ok) tc_commit(BAR(B_DONE));
      if (!ok) {
        atomicMax(status, ERR_BWD_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3, g = (warp - 2) >> 2;  // group g takes the key sub-tiles j = g, g + 3, ...
    const int row = quarter * 32 + lane;                // query row of this thread
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int q_idx = q0 + row;
    const bool q_live = q_idx < si.q_len;
    const long long tok = (long long)si.q_start + q_idx;
    const float lse2 = q_live ? lse2g[(long long)h * total_q + tok] : INFINITY;
    const float dlt = q_live ? delta[(long long)h * total_q + tok] : 0.f;
    const float scale_log2 = scale * LOG2E;
    int limit = si.k_len;
    if (causal) limit = min(limit, q_idx + off + 1);
    bool ok = true;
    for (int j = g; j < n_it; j += DQ_GROUPS) {
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(B_SF + g), (j / DQ_GROUPS) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (j * SUB + SUB > si.k_len) || (causal && j * SUB + SUB - 1 > q0 + off);
      uint32_t dpk[32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t s[32], dp[32];
        tc_ld32(t_lane + g * SUB + half * 32, s);
        tc_ld32(t_lane + (DQ_GROUPS + g) * SUB + half * 32, dp);
        tc_wait_ld();
        const int kbase = j * SUB + half * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2(fmaf(__uint_as_float(s[i]), scale_log2, -lse2));
          float p1 = ex2(fmaf(__uint_as_float(s[i + 1]), scale_log2, -lse2));
          if (need_mask) {
            if (kbase + i >= limit) p0 = 0.f;
            if (kbase + i + 1 >= limit) p1 = 0.f;
          }
          dpk[half * 16 + (i >> 1)] = pack2(p0 * (__uint_as_float(dp[i]) - dlt), p1 * (__uint_as_float(dp[i + 1]) - dlt));
        }
      }
      // dS goes back into tensor memory over the first 32 columns of this group's dP buffer and is the A operand of the dQ MMAs
      tc_st32(t_lane + (DQ_GROUPS + g) * SUB, dpk);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_DF + g));
    }
    if (ok && n_it > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(B_DONE), 0, abort_flag));
      if (ok) tc_fence_after();
    }
    if (ok) {
      // the 32-column chunks of the accumulator row are shared out over the three groups
      constexpr int NCH = D / 32;
      const int c_begin = g == 0 ? 0 : (NCH == 4 ? g + 1 : g), c_end = g == 0 ? (NCH == 4 ? 2 : 1) : min(NCH, c_begin + 1);
      store_acc_row(t_lane + 2 * DQ_GROUPS * SUB, dQ + tok * dq_row_stride + (long long)h * D, q_live, n_it > 0, c_begin, c_end, scale);
    } else if (lane == 0) {
      atomicMax(status, ERR_BWD_ROWS);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

template <int D>
int launch_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
               float* delta, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k, int batch, int sq, int sk,
               int max_q, int max_k, long long total_q, long long total_k, int Hq, int Hkv, long long q_rs, long long k_rs,
               long long v_rs, long long o_rs, long long do_rs, long long dq_rs, long long dk_rs, float scale, bool causal,
               int* status, cudaStream_t st, const CpAttn& cp) {
  CUtensorMap mq64, mdo64, mk128, mv128, mq128, mdo128, mk64, mv64;
  bool ok = cache().get(&mq64, q, (long long)Hq * D, total_q, q_rs, 64, 64) &&
            cache().get(&mdo64, dout, (long long)Hq * D, total_q, do_rs, 64, 64) &&
            cache().get(&mk128, k, (long long)Hkv * D, total_k, k_rs, 64, 128) &&
            cache().get(&mv128, v, (long long)Hkv * D, total_k, v_rs, 64, 128) &&
            cache().get(&mq128, q, (long long)Hq * D, total_q, q_rs, 64, 128) &&
            cache().get(&mdo128, dout, (long long)Hq * D, total_q, do_rs, 64, 128) &&
            cache().get(&mk64, k, (long long)Hkv * D, total_k, k_rs, 64, 64) &&
            cache().get(&mv64, v, (long long)Hkv * D, total_k, v_rs, 64, 64);
  if (!ok) return -1000 - g_last_map_error;
  auto kern_a = flash_bwd_dkdv_kernel<D>;
  auto kern_b = flash_bwd_dq_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern_a, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<D>::SMEM) != cudaSuccess) return -4;
    if (cudaFuncSetAttribute(kern_b, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<D>::SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  const long long warps = (total_q * Hq + (32 / (D / 8)) - 1) / (32 / (D / 8));
  float* lse2 = delta + total_q * Hq;  // second half of the scratch: lse in log2 units
  flash_delta_kernel<D><<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, lse, delta, lse2, total_q, Hq, do_rs, o_rs);
  const dim3 grid_a(Hkv * batch, (max_k + 127) / 128, 1);
  kern_a<<<grid_a, BWD_THREADS, DkvCfg<D>::SMEM, st>>>(mq64, mdo64, mk128, mv128, lse2, delta, (__nv_bfloat16*)dk,
                                                       (__nv_bfloat16*)dv, cu_q, cu_k, sq, sk, Hq, Hkv, dk_rs, total_q,
                                                       scale, causal ? 1 : 0, status, cp);
  const dim3 grid_b(Hq * batch, (max_q + 127) / 128, 1);
  kern_b<<<grid_b, DQ_THREADS, DqCfg<D>::SMEM, st>>>(mq128, mdo128, mk64, mv64, lse2, delta, (__nv_bfloat16*)dq, cu_q,
                                                      cu_k, sq, sk, Hq, Hkv, dq_rs, total_q, scale, causal ? 1 : 0, status, cp);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
              float* delta, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k, int batch, int sq, int sk,
              int max_q, int max_k, long long total_q, long long total_k, int Hq, int Hkv, int D, long long q_rs,
              long long k_rs, long long v_rs, long long o_rs, long long do_rs, long long dq_rs, long long dk_rs, float scale,
              bool causal, int* status, cudaStream_t st, const CpAttn* cp_in) {
  if (batch <= 0 || total_q <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv) return -1;
  CpAttn cp;
  if (cp_in != nullptr && cp_in->world > 1) {
    cp = *cp_in;
    if (cu_q || cu_k || !causal || cp.world > 8 || cp.rank < 0 || cp.rank >= cp.world) return -8;
    if (cp.chunk <= 0 || cp.chunk % 128 || sq != 2 * cp.chunk || sk != 2 * cp.world * cp.chunk) return -8;
    if (cp.k_vis != (2 * cp.world - cp.rank) * cp.chunk || max_k != cp.k_vis) return -8;
    if (cp.stage[0] != nullptr && cp.tile_counter == nullptr) return -9;
    cp.batch = batch;
  }
  if (D == 128)
    return launch_bwd<128>(q, k, v, out, dout, lse, delta, dq, dk, dv, cu_q, cu_k, batch, sq, sk, max_q, max_k, total_q,
                           total_k, Hq, Hkv, q_rs, k_rs, v_rs, o_rs, do_rs, dq_rs, dk_rs, scale, causal, status, st, cp);
  if (D == 64)
    return launch_bwd<64>(q, k, v, out, dout, lse, delta, dq, dk, dv, cu_q, cu_k, batch, sq, sk, max_q, max_k, total_q,
                          total_k, Hq, Hkv, q_rs, k_rs, v_rs, o_rs, do_rs, dq_rs, dk_rs, scale, causal, status, st, cp);
  return -3;
}

int cp_dkv_reduce(void* dk_local, void* dv_local, int batch, int row_elems, const CpAttn& cp_in, int* status, cudaStream_t st) {
  if (cp_in.world <= 1 || cp_in.stage[0] == nullptr || row_elems % 8 || batch <= 0) return -1;
  CpAttn cp = cp_in;
  cp.batch = batch;
  const long long total = 2LL * batch * 2 * cp.chunk * (row_elems / 8);
  const long long want = (total + 255) / 256;
  const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
  cp_dkv_reduce_kernel<<<blocks, 256, 0, st>>>((__nv_bfloat16*)dk_local, (__nv_bfloat16*)dv_local, row_elems, cp, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ab
