// Flash attention forward on tcgen05 (sm_100a): O = softmax(scale * Q K^T + mask) V, fp32 accumulation in TMEM.
//
// One CTA per (128-row Q tile, query head, sequence); 6 warps with fixed roles:
//   warp 0     : TMA producer - Q tile once, then K and V tiles of 128 keys through two 2-stage rings
//   warp 1     : MMA issuer   - S(j) = Q K(j)^T into one of two TMEM score buffers, O += P(j) V(j) into the TMEM
//                output accumulator; S(j+1) is issued BEFORE waiting for P(j), so the tensor cores work on the next
//                scores while the softmax warps are busy with the current ones
//   warps 2..5 : softmax + epilogue - one thread per query row: tcgen05.ld of the 128 scores of its row (no
//                shuffles), running max / sum in the exp2 domain, bf16 probabilities written to shared memory in
//                the 128-byte-swizzled K-major layout the PV MMA reads, O rescaled in TMEM only when the running
//                max grew by more than 2^8 (the stale max is exact after the final 1/l normalisation)
// Layouts: tokens are packed along the first dim, q [Tq, Hq, D], k/v [Tk, Hkv, D] (unit stride in D, heads adjacent);
// sequences are given by cu_seqlens (varlen) or a fixed length (dense).  Causal masking is lower-right aligned
// (query i of a sequence sees keys <= i + k_len - q_len), which covers training (k_len == q_len) and prefill on top
// of a cached prefix.  GQA: query head h reads kv head h / (Hq / Hkv).
// Takes the place of F.scaled_dot_product_attention / flash_attn in the reference's training and prefill paths
// (astrai/extension/backend/attention.py:453-468, 663-669) and of its mma.sync prefill kernel
// (csrc/kernels/attention/prefill_split_q_mma.cuh:19-157).
// Context parallel (CpAttn, world > 1): the keys are the gathered sequence; a few extra CTAs at the front of the grid
// pull every rank's K / V chunks from peer memory into the local gathered buffer (bulk copies through shared memory,
// ring order) and publish one flag per source rank, while the attention CTAs start with the chunks that are already
// local and poll the flag of a chunk's owner before its first TMA load - gather and attention are ONE launch.
// Every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, records a code in `status`,
// and all roles fall through to the common exit where TMEM is freed.
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

constexpr int BQ = 128, BKV = 64, FA_THREADS = 192, KV_STAGES = 2;
constexpr int BLK_BYTES = 128 * 128;   // one [128 rows x 64 bf16] swizzled block (Q, P)
constexpr int KBLK_BYTES = BKV * 128;  // one [64 rows x 64 bf16] swizzled block (K, V)
enum : int { ERR_FA_PRODUCER = 31, ERR_FA_MMA = 32, ERR_FA_SOFTMAX = 33 };

template <int D>
struct FwdCfg {
  static constexpr int NB = D / 64;
  static constexpr int TILE_BYTES = 128 * D * 2;   // Q tile
  static constexpr int KV_BYTES = BKV * D * 2;     // one K or V stage
  static constexpr int P_BYTES = 128 * BKV * 2;
  // Two CTAs share an SM (each holds 256 TMEM columns), so a CTA may use half of the SM's shared memory minus the
  // per-CTA reservation: 115 712 bytes at head dim 128, which leaves 768 bytes for aligning the tiles to 1024.
  static constexpr int ALIGN_SLACK = 768;
  static constexpr int SMEM = TILE_BYTES + 2 * KV_STAGES * KV_BYTES + P_BYTES + 256 + ALIGN_SLACK;
};

struct SeqInfo {
  int q_start, q_len, k_start, k_len;
};
__device__ __forceinline__ SeqInfo seq_info(const int* cu_q, const int* cu_k, int b, int sq, int sk) {
  SeqInfo s;
  s.q_start = cu_q ? cu_q[b] : b * sq;
  s.q_len = cu_q ? cu_q[b + 1] - cu_q[b] : sq;
  s.k_start = cu_k ? cu_k[b] : b * sk;
  s.k_len = cu_k ? cu_k[b + 1] - cu_k[b] : sk;
  return s;
}

// Gather CTA (one thread works): announce that this rank's K / V source is complete, then, for every source rank in
// ring order starting with this one, wait (bounded) for its announcement and move this CTA's share of its four
// segments (K | V) x (first | second chunk) per batch entry into the gathered buffers: up to NS pieces of 32 KB are in
// flight through shared memory at a time.  The last CTA to finish a source rank publishes chunk_flags[src] = epoch.
template <int SMEM_BYTES>
__device__ void gather_kv(const CpAttn& cp, int cta, int row_bytes, int* status) {
  constexpr int PIECE = 32768;
  constexpr int NS = (SMEM_BYTES - 1024 - 256) / PIECE;
  static_assert(NS >= 1, "no room for a copy slot");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + NS * PIECE);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NS);
  const uint32_t bar0 = smem_u32(bars);
  for (int s = 0; s < NS; ++s) mbar_init(bar0 + 8u * s, 1);
  *abort_flag = 0;
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  fence_async_smem();

  const int W = cp.world, r = cp.rank, n_copy = cp.n_copy_ctas;
  if (cta == 0) {
    __threadfence_system();
    for (int p = 0; p < W; ++p) comm::st_release_sys(flag_slot(cp.flags[p], KIND_CP_KV, r, cp.unit, cp.max_units), cp.epoch);
  }
  const long long seg_bytes = (long long)cp.chunk * row_bytes;
  const int pps = (int)((seg_bytes + PIECE - 1) / PIECE);  // pieces per segment
  const int total = 4 * cp.batch * pps;
  const long long S = 2LL * W * cp.chunk;
  uint32_t phase = 0;
  for (int i = 0; i < W; ++i) {
    const int src = (r + i) % W;
    if (i > 0 && !comm::wait_flag(flag_slot(cp.flags[r], KIND_CP_KV, src, cp.unit, cp.max_units), cp.epoch, cp.timeout_ns)) {
      atomicMax(status, ERR_CP_COPY);
      return;  // the attention CTAs run out of time on the chunk flag and report as well
    }
    const uint8_t* from = reinterpret_cast<const uint8_t*>(cp.kv_src[src]);
    for (int first = cta; first < total; first += n_copy * NS) {
      uint8_t* dst[NS];
      uint32_t bytes[NS];
      int n = 0;
      for (; n < NS; ++n) {
        const int pc = first + n * n_copy;
        if (pc >= total) break;
        const int seg = pc / pps, pi = pc % pps;
        const int kv = seg / (2 * cp.batch), b = (seg >> 1) % cp.batch, half = seg & 1;
        const long long src_off = (((long long)kv * cp.batch + b) * 2 + half) * seg_bytes + (long long)pi * PIECE;
        const long long dst_off = ((long long)b * S + (long long)chunk_of(src, half, W) * cp.chunk) * row_bytes + (long long)pi * PIECE;
        dst[n] = reinterpret_cast<uint8_t*>(kv ? cp.v_full : cp.k_full) + dst_off;
        bytes[n] = (uint32_t)min((long long)PIECE, seg_bytes - (long long)pi * PIECE);
        mbar_expect_tx(bar0 + 8u * n, bytes[n]);
        bulk_load(base + n * PIECE, from + src_off, bytes[n], bar0 + 8u * n);
      }
      for (int s = 0; s < n; ++s) {
        if (!mbar_wait(bar0 + 8u * s, phase, abort_flag)) {
          atomicMax(status, ERR_CP_COPY);
          return;
        }
        bulk_store(dst[s], base + s * PIECE, bytes[s]);
      }
      // barriers of unused slots did not flip: give them the phase the used ones have now
      for (int s = n; s < NS; ++s) {
        mbar_arrive(bar0 + 8u * s);
        if (!mbar_wait(bar0 + 8u * s, phase, abort_flag)) return;
      }
      bulk_commit();
      bulk_wait_read();  // the slots may be overwritten
      phase ^= 1u;
    }
    bulk_wait_all();  // every store of this source rank has landed
    fence_async_global();
    __threadfence();
    const int done = atomicAdd(&cp.chunk_counter[src], 1);
    if (done == n_copy - 1) {
      cp.chunk_counter[src] = 0;
      st_release_gpu(&cp.chunk_flags[src], cp.epoch);
    }
  }
}

// One unit of work of the persistent forward kernel: a 128-row query tile of one head of one sequence.
struct FwdItem {
  SeqInfo si;
  int h, kvh, q0, off, n_kv, b;
};
// Work items are numbered heaviest first: item w covers (head x sequence) w % nbx and the (w / nbx)-th query tile counted
// from the end of the sequence (under a causal mask the last tile sees the most keys).  Returns false when the sequence
// has no such tile.
__device__ __forceinline__ bool fwd_item(int w, int nbx, const int* cu_q, const int* cu_k, int sq, int sk, int Hq, int Hkv,
                                         int causal, const CpAttn& cp, FwdItem& im) {
  const int bx = w % nbx, by = w / nbx;
  im.h = bx % Hq;
  im.b = bx / Hq;
  im.si = seq_info(cu_q, cu_k, im.b, sq, sk);
  if (cp.world > 1) im.si.k_len = cp.k_vis;
  const int qt = (im.si.q_len + BQ - 1) / BQ - 1 - by;
  if (qt < 0) return false;
  im.kvh = im.h / (Hq / Hkv);
  im.q0 = qt * BQ;
  im.off = (cp.world > 1 && im.q0 < cp.chunk) ? cp.rank * cp.chunk : im.si.k_len - im.si.q_len;
  int kv_end = im.si.k_len;
  if (causal) kv_end = min(im.si.k_len, im.q0 + BQ + im.off);
  if (kv_end < 0) kv_end = 0;
  im.n_kv = (kv_end + BKV - 1) / BKV;
  return true;
}

// Persistent kernel, two CTAs per SM: each walks over its share of the work items (round k: item k * P + c for even k,
// k * P + P - 1 - c for odd k, which evens out the heaviest-first list across the P CTAs).  A CTA works on 128 x 64
// score tiles with half of the SM's shared memory and 256 TMEM columns (S0 | S1 | O); while one CTA's four softmax
// warps hold the exponential unit, the other CTA's MMAs, loads, barriers and epilogue fill in.  All barrier phases run
// on counters that continue across items.
template <int D>
__global__ void __launch_bounds__(FA_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ O, float* __restrict__ lse,
                 const int* __restrict__ cu_q, const int* __restrict__ cu_k, int sq, int sk, int Hq, int Hkv, int nbx,
                 int n_items, long long o_row_stride, long long total_q, float scale_log2, int causal,
                 int* __restrict__ status, const CpAttn cp, const PagedKv pg) {
  using C = FwdCfg<D>;
  const bool gather = cp.world > 1 && cp.kv_src[0] != nullptr;
  const int n_copy = gather ? cp.n_copy_ctas : 0;
  if ((int)blockIdx.x < n_copy) {
    if (threadIdx.x == 0) gather_kv<C::SMEM>(cp, (int)blockIdx.x, Hkv * D * 2, status);
    return;
  }
  const int P = (int)gridDim.x - n_copy, cta = (int)blockIdx.x - n_copy;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  if (base - smem_u32(smem_raw) > (uint32_t)C::ALIGN_SLACK) {  // cannot happen while dynamic shared memory starts 1024-aligned
    if (threadIdx.x == 0) atomicMax(status, ERR_FA_PRODUCER);
    return;
  }
  const uint32_t q_smem = base;
  const uint32_t k_smem = base + C::TILE_BYTES;
  const uint32_t v_smem = k_smem + KV_STAGES * C::KV_BYTES;
  const uint32_t p_smem = v_smem + KV_STAGES * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (p_smem - base) + C::P_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  enum : int { QF = 0, QE = 1, KF = 2, KE = 4, VF = 6, VE = 8, SF = 10, PF = 12, PE = 13, OE = 14, NBAR = 15 };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < NBAR; ++i) mbar_init(BAR(i), (i == PF || i >= OE) ? 4 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(256u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;  // columns: S0 (64) | S1 (64) | O (128)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      uint32_t tq = 0, kc = 0;
      uint32_t landed = 0;  // source ranks whose chunks are known to be in the gathered buffer
      for (int k = 0; k * P < n_items && ok; ++k) {
        const int w = k * P + ((k & 1) ? P - 1 - cta : cta);
        FwdItem im;
        if (w >= n_items || !fwd_item(w, nbx, cu_q, cu_k, sq, sk, Hq, Hkv, causal, cp, im) || im.n_kv == 0) continue;
        if (!mbar_wait(BAR(QE), (tq & 1) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(BAR(QF), C::TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < C::NB; ++kb)
          tma_load_2d(q_smem + kb * BLK_BYTES, &map_q, BAR(QF), im.h * D + kb * 64, im.si.q_start + im.q0);
        KvOrder order(im.n_kv, cp, BKV);
        for (int it = 0; it < im.n_kv && ok; ++it, ++kc) {
          const int j = order.next();
          const uint32_t st = kc & 1;
          const uint32_t ph = ((kc >> 1) & 1) ^ 1u;
          if (gather) {
            const int owner = chunk_owner(j * BKV / cp.chunk, cp.world);
            if (!((landed >> owner) & 1u)) {
              const unsigned long long t0 = comm::now_ns();
              while (ld_acquire_gpu(&cp.chunk_flags[owner]) < cp.epoch) {
                if (*abort_flag || comm::now_ns() - t0 > cp.timeout_ns) { ok = false; break; }
                __nanosleep(100);
              }
              if (!ok) { atomicMax(status, ERR_CP_CHUNK_WAIT); break; }
              fence_async_global();
              landed |= 1u << owner;
            }
          }
          if (!mbar_wait(BAR(KE + st), ph, abort_flag)) { ok = false; break; }
          mbar_expect_tx(BAR(KF + st), C::KV_BYTES);
          if (pg.table == nullptr) {
#pragma unroll
            for (int kb = 0; kb < C::NB; ++kb)
              tma_load_2d(k_smem + st * C::KV_BYTES + kb * KBLK_BYTES, &map_k, BAR(KF + st), im.kvh * D + kb * 64, im.si.k_start + j * BKV);
          }
          // Paged pool: the tile's keys live in 64 / page pages; each page is `page` consecutive pool rows whose first
          // slot the table names.  Pages past the end of the sequence load slot 0 (their scores are masked anyway).
          int slot_of[BKV / 8];
          if (pg.table != nullptr) {
            const int* trow = pg.table + (long long)pg.rows[im.b] * pg.stride;
            const int subs = BKV / pg.page;
            for (int sp = 0; sp < subs; ++sp) {
              const int t = j * BKV + sp * pg.page;
              slot_of[sp] = t < im.si.k_len ? trow[t] : 0;
            }
            for (int sp = 0; sp < subs; ++sp)
#pragma unroll
              for (int kb = 0; kb < C::NB; ++kb)
                tma_load_2d(k_smem + st * C::KV_BYTES + kb * KBLK_BYTES + sp * pg.page * 128, &map_k, BAR(KF + st),
                            im.kvh * D + kb * 64, slot_of[sp]);
          }
          if (!mbar_wait(BAR(VE + st), ph, abort_flag)) { ok = false; break; }
          mbar_expect_tx(BAR(VF + st), C::KV_BYTES);
          if (pg.table == nullptr) {
#pragma unroll
            for (int kb = 0; kb < C::NB; ++kb)
              tma_load_2d(v_smem + st * C::KV_BYTES + kb * KBLK_BYTES, &map_v, BAR(VF + st), im.kvh * D + kb * 64, im.si.k_start + j * BKV);
          } else {
            const int subs = BKV / pg.page;
            for (int sp = 0; sp < subs; ++sp)
#pragma unroll
              for (int kb = 0; kb < C::NB; ++kb)
                tma_load_2d(v_smem + st * C::KV_BYTES + kb * KBLK_BYTES + sp * pg.page * 128, &map_v, BAR(VF + st),
                            im.kvh * D + kb * 64, slot_of[sp]);
          }
        }
        ++tq;
      }
      if (!ok) {
        atomicMax(status, ERR_FA_PRODUCER);
        *abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, BKV, false, false);
      constexpr uint32_t idesc_pv = idesc_bf16(128, D, false, true);
      const uint32_t q_lo0 = desc_lo(q_smem, true, 0), k_lo0 = desc_lo(k_smem, true, 0);
      const uint32_t v_lo0 = desc_lo(v_smem, false, KBLK_BYTES);
      bool ok = true;
      uint32_t tq = 0, kc = 0;
      bool have_prev = false, prev_first = false;
      uint32_t prev_kc = 0, prev_tq = 0;
      // O += P V of tile `prev`: its P must be in shared memory, its V landed, and (first tile of an item) the epilogue
      // that last used this O buffer must have read it.
      auto issue_pv = [&]() -> bool {
        const uint32_t st = prev_kc & 1;
        if (!mbar_wait(BAR(PF), prev_kc & 1, abort_flag) || !mbar_wait(BAR(VF + st), (prev_kc >> 1) & 1, abort_flag)) return false;
        if (prev_first && prev_tq >= 1 && !mbar_wait(BAR(OE), (prev_tq - 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t v_lo = v_lo0 + st * (C::KV_BYTES >> 4);
        const uint32_t d = tmem_base + 128;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          tc_mma_ts(d, tmem_base + st * BKV + 8 * k, v_lo + k * 128, idesc_pv, (!prev_first || k) ? 1u : 0u);
        tc_commit(BAR(VE + st));  // V stage free
        tc_commit(BAR(PE));       // P consumed, O updated
        return true;
      };
      for (int k = 0; k * P < n_items && ok; ++k) {
        const int w = k * P + ((k & 1) ? P - 1 - cta : cta);
        FwdItem im;
        if (w >= n_items || !fwd_item(w, nbx, cu_q, cu_k, sq, sk, Hq, Hkv, causal, cp, im) || im.n_kv == 0) continue;
        if (!mbar_wait(BAR(QF), tq & 1, abort_flag)) { ok = false; break; }
        const uint32_t q_lo = q_lo0;
        for (int j = 0; j < im.n_kv; ++j, ++kc) {
          // scores of tile kc first, then the P V product of the tile before it: the softmax of one tile overlaps the
          // score MMAs of the next, also across item boundaries
          const uint32_t st = kc & 1;
          if (!mbar_wait(BAR(KF + st), (kc >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + st * BKV;
          const uint32_t k_lo = k_lo0 + st * (C::KV_BYTES >> 4);
#pragma unroll
          for (int kb = 0; kb < C::NB; ++kb)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma_lo(d, q_lo + kb * (BLK_BYTES >> 4) + 2 * kk, k_lo + kb * (KBLK_BYTES >> 4) + 2 * kk, idesc_s, (kb | kk) ? 1u : 0u);
          tc_commit(BAR(KE + st));                         // K stage free
          if (j == im.n_kv - 1) tc_commit(BAR(QE));        // last use of this Q tile
          tc_commit(BAR(SF + st));                         // scores ready
          if (have_prev && !issue_pv()) { ok = false; break; }
          have_prev = true;
          prev_first = j == 0;
          prev_kc = kc;
          prev_tq = tq;
        }
        ++tq;
      }
      if (ok && have_prev) ok = issue_pv();
      if (!ok) {
        atomicMax(status, ERR_FA_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (one thread per row)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    uint32_t tq = 0, kc = 0;
    for (int k = 0; k * P < n_items && ok; ++k) {
      const int w = k * P + ((k & 1) ? P - 1 - cta : cta);
      FwdItem im;
      if (w >= n_items || !fwd_item(w, nbx, cu_q, cu_k, sq, sk, Hq, Hkv, causal, cp, im)) continue;
      const SeqInfo& si = im.si;
      const int q0 = im.q0, off = im.off, n_kv = im.n_kv, h = im.h;
      const int q_idx = q0 + row;
      const bool live = q_idx < si.q_len;
      const long long tok = (long long)si.q_start + q_idx;
      __nv_bfloat16* orow = O + tok * o_row_stride + (long long)h * D;
      if (n_kv == 0) {  // no visible key: zero output, lse = -inf
        if (live) {
#pragma unroll 1
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0u, 0u, 0u, 0u);
          if (lse != nullptr) lse[(long long)h * total_q + tok] = -INFINITY;
        }
        continue;
      }
      const uint32_t t_o = t_lane + 128;
      float m_run = -INFINITY, l_run = 0.f;
      KvOrder order(n_kv, cp, BKV);
      for (int it = 0; it < n_kv; ++it, ++kc) {
        const int j = order.next();
        const uint32_t buf = kc & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(BAR(SF + buf), (kc >> 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        uint32_t s[2][32];
#pragma unroll
        for (int c = 0; c < 2; ++c) tc_ld32(t_lane + buf * BKV + c * 32, s[c]);
        tc_wait_ld();
        const int k0 = j * BKV;
        const bool need_mask = (k0 + BKV > si.k_len) || (causal && (k0 + BKV - 1 > q0 + off));
        if (need_mask) {
          int limit = si.k_len;
          if (causal) limit = min(limit, q_idx + off + 1);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (k0 + c * 32 + i >= limit) s[c][i] = __float_as_uint(-INFINITY);
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains: a single warp needs the ILP
#pragma unroll
        for (int i = 0; i < 32; i += 2)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            mx4[2 * c] = fmaxf(mx4[2 * c], __uint_as_float(s[c][i]));
            mx4[2 * c + 1] = fmaxf(mx4[2 * c + 1], __uint_as_float(s[c][i + 1]));
          }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_new = fmaxf(m_run, mx * scale_log2);
        const bool grow = __any_sync(0xffffffffu, m_new > m_run + 8.f);
        float alpha = 1.f, m_use = m_run;
        if (grow) {
          m_use = m_new;
          alpha = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_new);
        }
        const float m_safe = (m_use == -INFINITY) ? 0.f : m_use;
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float p0 = ex2(fmaf(__uint_as_float(s[c][i]), scale_log2, -m_safe));
            const float p1 = ex2(fmaf(__uint_as_float(s[c][i + 1]), scale_log2, -m_safe));
            rs4[2 * c] += p0;
            rs4[2 * c + 1] += p1;
            const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
            pk[c * 16 + (i >> 1)] = *reinterpret_cast<const uint32_t*>(&hh);
          }
        const float rowsum = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        if (kc > 0) {
          // Every tile observes the completion of the previous P V product, needed or not: a parity wait is only
          // sound while the waiter is at most one phase behind the barrier, and the end-of-item wait below relies on it.
          ok = __all_sync(0xffffffffu, mbar_wait(BAR(PE), (kc - 1) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (it > 0 && grow) {  // that product has updated O, which may now be rescaled
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tc_ld32(t_o + c * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tc_st32(t_o + c * 32, o);
            }
            tc_wait_st();
          }
        }
        l_run = l_run * alpha + rowsum;
        m_run = m_use;
        // P row -> tensor memory, over the first 32 columns of this tile's score buffer (the scores are in registers by
        // now): the P V product reads it as its A operand, and the score MMAs of tile kc + 2, issued after that product
        // by the same thread, overwrite it in order.
        tc_st32(t_lane + buf * BKV, pk);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(PF));
      }
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(PE), (kc - 1) & 1, abort_flag));  // last P V of the item: O complete
      if (!ok) break;
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tc_ld32(t_o + c * 32, o);
        tc_wait_ld();
        if (live) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 pkd;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pkd);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o[8 * v4 + 2 * q]) * inv_l,
                                                              __uint_as_float(o[8 * v4 + 2 * q + 1]) * inv_l);
              pw[q] = *reinterpret_cast<const uint32_t*>(&hh);
            }
            reinterpret_cast<uint4*>(orow + c * 32)[v4] = pkd;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(OE));  // O may be overwritten
      if (live && lse != nullptr)
        lse[(long long)h * total_q + tok] = (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      ++tq;
    }
    if (!ok && lane == 0) {
      atomicMax(status, ERR_FA_SOFTMAX);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

template <int D>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* O, float* lse, const int* cu_q,
               const int* cu_k, int batch, int sq, int sk, int max_q, int Hq, int Hkv, long long o_row_stride,
               long long total_q, float scale, bool causal, int* status, cudaStream_t st, const CpAttn& cp,
               const PagedKv& pg) {
  auto kern = flash_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<D>::SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  const int n_copy = (cp.world > 1 && cp.kv_src[0] != nullptr) ? cp.n_copy_ctas : 0;
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0)
      n_sm = 148;
  }
  // two resident CTAs per SM: copy CTAs (context parallel) and persistent attention CTAs together fill the GPU once
  const int nbx = Hq * batch, n_items = nbx * ((max_q + BQ - 1) / BQ);
  int n_persist = 2 * n_sm - n_copy;
  if (n_persist < 1) n_persist = 1;
  if (n_persist > n_items) n_persist = n_items;
  const dim3 grid(n_persist + n_copy, 1, 1);
  kern<<<grid, FA_THREADS, FwdCfg<D>::SMEM, st>>>(mq, mk, mv, (__nv_bfloat16*)O, lse, cu_q, cu_k, sq, sk, Hq, Hkv, nbx, n_items,
                                                  o_row_stride, total_q, scale * 1.4426950408889634f, causal ? 1 : 0,
                                                  status, cp, pg);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q, const int* cu_k,
              int batch, int sq, int sk, int max_q, long long total_q, long long total_k, int Hq, int Hkv, int D,
              long long q_row_stride, long long k_row_stride, long long v_row_stride, long long o_row_stride, float scale,
              bool causal, int* status, cudaStream_t st, const CpAttn* cp_in, const PagedKv* paged) {
  if (batch <= 0 || total_q <= 0) return 0;
  PagedKv pg;
  if (paged != nullptr && paged->table != nullptr) {
    pg = *paged;
    // the key counts must come from cu_k; a page is a whole number of 8-row swizzle atoms and divides the 64-key tile
    if (!cu_k || !pg.rows || pg.stride <= 0 || (pg.page != 8 && pg.page != 16 && pg.page != 32 && pg.page != 64)) return -10;
    if (cp_in != nullptr && cp_in->world > 1) return -10;
  }
  if (Hkv <= 0 || Hq % Hkv) return -1;
  if (D != 64 && D != 128) return -3;
  CpAttn cp;
  if (cp_in != nullptr && cp_in->world > 1) {
    cp = *cp_in;
    // dense causal only; chunks are whole key tiles; the local rows are the rank's two chunks
    if (cu_q || cu_k || !causal || cp.world > 8 || cp.rank < 0 || cp.rank >= cp.world) return -8;
    if (cp.chunk <= 0 || cp.chunk % BKV || sq != 2 * cp.chunk || sk != 2 * cp.world * cp.chunk) return -8;
    if (cp.k_vis != (2 * cp.world - cp.rank) * cp.chunk) return -8;
    if (cp.kv_src[0] != nullptr) {
      if (cp.n_copy_ctas < 1 || cp.n_copy_ctas > 32 || !cp.k_full || !cp.v_full || !cp.chunk_flags || !cp.chunk_counter) return -9;
      if (k != cp.k_full || v != cp.v_full || k_row_stride != (long long)Hkv * D || v_row_stride != k_row_stride) return -9;
      cp.batch = batch;
    }
  }
  CUtensorMap mq, mk, mv;
  if (!cache().get(&mq, q, (long long)Hq * D, total_q, q_row_stride, 64, 128)) return -1000 - g_last_map_error;
  const int kv_box_rows = pg.table != nullptr ? pg.page : BKV;
  if (!cache().get(&mk, k, (long long)Hkv * D, total_k, k_row_stride, 64, kv_box_rows)) return -2000 - g_last_map_error;
  if (!cache().get(&mv, v, (long long)Hkv * D, total_k, v_row_stride, 64, kv_box_rows)) return -3000 - g_last_map_error;
  if (D == 128)
    return launch_fwd<128>(mq, mk, mv, out, lse, cu_q, cu_k, batch, sq, sk, max_q, Hq, Hkv, o_row_stride, total_q, scale,
                           causal, status, st, cp, pg);
  return launch_fwd<64>(mq, mk, mv, out, lse, cu_q, cu_k, batch, sq, sk, max_q, Hq, Hkv, o_row_stride, total_q, scale,
                        causal, status, st, cp, pg);
}

}  // namespace ab
