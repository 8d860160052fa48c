// Host-callable launchers of the CUDA kernels.  No torch types here: the binding file converts tensors to
// pointers, so the .cu files compile in seconds and can be linked into other hosts.
#pragma once
#include <cuda_runtime.h>

namespace ab {

// `res` / `xsum` (wide rows only: cols % 8 == 0, 512 <= cols <= 16384): normalise x + res and write the sum to xsum.
void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                 bool is_bf16, cudaStream_t st, const void* res = nullptr, void* xsum = nullptr);
bool rmsnorm_wide(int cols);
int rmsnorm_bwd_parts(long long rows, int cols);
// `gres` (wide rows only): a second gradient of x, added into dx.
void rmsnorm_bwd(const void* g, const void* x, const void* w, const float* rstd, void* dx, float* dw, float* partial,
                 long long rows, int cols, bool is_bf16, cudaStream_t st, const void* gres = nullptr);
void rope_apply(const void* x, void* out, const float* freqs, long long tokens, int heads, int rot_dim,
                long long x_tok_stride, int x_head_stride, long long o_tok_stride, int o_head_stride, bool inverse,
                bool is_bf16, cudaStream_t st);
void swiglu_fwd(const void* gate, const void* up, void* y, long long rows, int f, long long in_stride, bool is_bf16,
                cudaStream_t st);
void swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup, long long rows, int f,
                long long in_stride, long long out_stride, bool is_bf16, cudaStream_t st);
void embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int dim, long long vocab,
                   bool is_bf16, cudaStream_t st);
void embedding_bwd(const long long* ids, const void* g, float* grad_table, long long tokens, int dim, long long vocab,
                   bool is_bf16, cudaStream_t st);
// Deterministic variant: ids sorted ascending with the permutation that sorted them; equal ids are summed in run order.
void embedding_bwd_sorted(const long long* sorted, const long long* perm, const void* g, float* grad_table, long long tokens,
                          int dim, long long vocab, bool is_bf16, cudaStream_t st);

void ce_rows(const void* logits, void* dlogits, const long long* targets, float* loss, float* logprob,
             const float* grad_scale, long long rows, int V, long long ld, float smoothing, long long ignore_index,
             bool is_bf16, cudaStream_t st);
void logprob_bwd(const void* logits, void* dlogits, const long long* targets, const float* logprob,
                 const float* g_rows, long long rows, int V, long long ld, bool is_bf16, cudaStream_t st);
void sumsq_accum(const void* x, long long n, float* out, bool is_bf16, cudaStream_t st);
void clip_coef(const float* sumsq, float max_norm, float pre_scale, float* coef, float* norm_out, cudaStream_t st);
void adamw_step(void* p, float* master, float* g, float* m, float* v, long long n, float lr, float b1, float b2,
                float eps, float wd, int step, const float* gscale, bool zero_grad, bool p_bf16, cudaStream_t st);
void axpy_f32(float* dst, const void* src, long long n, float alpha, bool src_bf16, cudaStream_t st);

// Inference attention over a slot-addressed KV pool (paged_attention.cu).
void kv_append(const void* k_new, const void* v_new, void* k_buf, void* v_buf, const int* loc, long long tokens,
               int row_elems, long long n_slots, cudaStream_t st);
int paged_decode_splits(int batch, int n_kv_heads, long long max_len, int max_splits);
// k_new / v_new [batch, n_kv_heads, head_dim] (both or neither): fused append - the row of position seq_lens[b] - 1 is read
// from them and written into the pool slot the table names for that position (the pool is then written, not only read).
// table_rows: number of rows of req_to_token (a request whose req_pool_indices entry is outside [0, table_rows) attends to
// nothing), or 0 when the caller cannot say (raw-pointer entry points); seq_lens entries are cut to [0, max_ctx].
int paged_decode(const void* q, const void* k_buf, const void* v_buf, const int* req_to_token,
                 const int* req_pool_indices, const long long* seq_lens, float* o_part, float* ml_part, int* counters,
                 void* out, int batch, int n_q_heads, int n_kv_heads, int head_dim, int max_ctx, long long n_slots,
                 float scale, int splits, int max_splits, int table_rows, cudaStream_t st, const void* k_new = nullptr,
                 const void* v_new = nullptr);

// tcgen05 GEMM: D[M,N] (+)= A * B with bf16 operands and fp32 accumulation in tensor memory.
//   a_kmajor: A is [M,K] row-major (true) or stored as [K,M] row-major (false)
//   b_kmajor: B is [N,K] row-major (true) or stored as [K,N] row-major (false)
//   out_f32 : D is fp32 (else bf16); accumulate: D += result (read-modify-write in the epilogue)
// lda/ldb/ldd are row strides in elements of the stored matrices.  Returns 0, or a negative code on a bad argument.
int gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
              bool a_kmajor, bool b_kmajor, bool out_f32, bool accumulate, int* status, cudaStream_t st);

// Same contract, computed by CTA pairs (cta_group::2, 256x256 tiles).  Used by gemm_bf16 for M >= 256.
int gemm_bf16_2cta(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                   long long ldd, bool a_kmajor, bool b_kmajor, bool out_f32, bool accumulate, int* status,
                   cudaStream_t st);

// Context-parallel extension of the flash kernels.  The sequence of S = 2 * world * chunk tokens is cut into
// 2 * world chunks; rank r owns chunks r and 2 * world - 1 - r (zig-zag, so every rank has the same causal work).
// Its 2 * chunk local query rows attend to the gathered keys [0, k_vis), k_vis = (2 * world - r) * chunk: rows below
// `chunk` sit at global position r * chunk + i, the others at k_vis - 2 * chunk + i.  world == 1 switches all of it off.
struct CpAttn {
  int world = 1, rank = 0, chunk = 0, k_vis = 0, batch = 1;
  // forward gather, done by copy CTAs inside the attention kernel when kv_src[0] != null:
  const void* kv_src[8] = {};   // every rank's local [2 (k|v)][batch][2 * chunk][Hkv * D] bf16
  void* k_full = nullptr;       // local gathered [batch][S][Hkv * D]; the kernel's K / V operands
  void* v_full = nullptr;
  void* flags[8] = {};          // flag array of every rank ([kind][8][max_units] int32)
  int unit = 0, max_units = 1, epoch = 0, n_copy_ctas = 0;
  int* chunk_flags = nullptr;   // local int[8]: epoch at which rank p's chunks landed in k_full / v_full
  int* chunk_counter = nullptr; // local int[8]: copy CTAs finished per source rank (self-resetting)
  unsigned long long timeout_ns = 0;
  // backward scatter, done by the dK/dV epilogue when stage[0] != null:
  void* stage[8] = {};          // every rank's [world (src)][2 (dk|dv)][batch][2 * chunk][Hkv * D] bf16
  int* tile_counter = nullptr;  // local int[8]: tiles written per destination rank (self-resetting)
};

// Paged K / V for flash_fwd: prefill over a slot-addressed pool without gathering the keys first.  k / v are then the
// pool [n_slots, Hkv, D]; sequence b reads key t from slot table[rows[b] * stride + t]; the `page` tokens of one page
// (page in {8, 16, 32, 64}) sit in consecutive slots that start at a multiple of `page`, so a 64-key tile is 64 / page
// TMA loads of `page` rows each.  cu_k still gives the key counts (differences); its offsets are not used.
struct PagedKv {
  const int* table = nullptr;
  const int* rows = nullptr;
  long long stride = 0;
  int page = 0;
};

// Flash attention forward (flash_fwd.cu).  Packed layouts q [total_q, Hq, D], k/v [total_k, Hkv, D] with unit stride
// in D and adjacent heads; row strides in elements.  cu_q / cu_k: int32 [batch+1] sequence boundaries or null (then
// every sequence has sq / sk tokens).  lse [Hq, total_q] fp32 (natural log) may be null.  D in {64, 128}.
// With `cp` (world > 1): dense only, sq = 2 * chunk, sk = S, causal.
int flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q, const int* cu_k,
              int batch, int sq, int sk, int max_q, long long total_q, long long total_k, int Hq, int Hkv, int D,
              long long q_row_stride, long long k_row_stride, long long v_row_stride, long long o_row_stride, float scale,
              bool causal, int* status, cudaStream_t st, const CpAttn* cp = nullptr, const PagedKv* paged = nullptr);

// Flash attention backward (flash_bwd.cu): dq [total_q,Hq,D], dk/dv [total_k,Hkv,D] bf16; `delta` is fp32 scratch
// [2, Hq, total_q]; lse as written by flash_fwd.  Three launches: row-dot pre-pass, dK/dV kernel, dQ kernel.
// With `cp`: dk/dv are this rank's PARTIAL gradients of the gathered keys [batch][S] (rows from k_vis on are not
// written), or, when cp->stage is set, they are not used and every tile goes to its owner's staging slot.
int flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
              float* delta, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k, int batch, int sq, int sk,
              int max_q, int max_k, long long total_q, long long total_k, int Hq, int Hkv, int D, long long q_rs,
              long long k_rs, long long v_rs, long long o_rs, long long do_rs, long long dq_rs, long long dk_rs, float scale,
              bool causal, int* status, cudaStream_t st, const CpAttn* cp = nullptr);
// Owner side of the backward scatter: waits (bounded) for every contributing rank's tiles, then
// dk_local / dv_local [batch][2 * chunk][Hkv * D] = sum over the contributors' staging slots.
int cp_dkv_reduce(void* dk_local, void* dv_local, int batch, int row_elems, const CpAttn& cp, int* status, cudaStream_t st);

// ---- communication kernels over peer memory (comm_fsdp.cu, comm.cuh)
struct CommPeers { void* ptr[8]; };  // the same buffer on every rank of the node, indexed by rank

// Reduce-scatter of one flat gradient unit + squared-norm partial.  `grads.ptr[r]` is the unit's fp32 gradient buffer
// on rank r; the caller owns elements [shard_off, shard_off+n).  `mc_grads` (may be null) is the NVSwitch multicast
// address of the same buffer: when given, one multimem.ld_reduce replaces the per-rank loads.  `flags.ptr[r]` is the
// int32 flag array of rank r ([kind][8][max_units]).  `timeout_ns` bounds the wait for the peers' gradients.
int fsdp_reduce_scatter(const CommPeers& grads, const float* mc_grads, const CommPeers& flags, int world, int rank,
                        long long shard_off, long long n, float* out, float* sumsq, int unit, int max_units, int epoch,
                        unsigned long long timeout_ns, int* status, int max_ctas, cudaStream_t st);
// AdamW on the owned shard + store of the new bf16 parameters into every rank's parameter buffer + "written" flag.
int fsdp_adamw_allgather(const CommPeers& params, void* mc_params, const CommPeers& flags, int world, int rank,
                         long long shard_off, long long n, float* master, const float* g, float* m, float* v, float lr,
                         float b1, float b2, float eps, float wd, int step, const float* gscale, int unit,
                         int max_units, int epoch, int* block_counter, int max_ctas, cudaStream_t st);
// Wait (bounded) until every rank except `skip_rank` has published `epoch` for (kind, unit) in this rank's flag array.
int comm_wait_flags(const int* local_flags, int kind, int world, int skip_rank, int unit, int max_units, int epoch,
                    unsigned long long timeout_ns, int* status, cudaStream_t st);

// ---- tensor-parallel GEMMs fused with their collective (gemm_comm.cu)
struct TpGemmParams {
  int world, rank, unit, max_units, epoch, n_copy_ctas, fuse_reduce;
  unsigned long long timeout_ns;
  void* flags[8];        // flag array of every rank ([kind][8][max_units] int32)
  void* x_full[8];       // all-gather: the [M, K] activation buffer of every rank (rank r owns row block r of its own)
  int* chunk_flags;      // all-gather, local int[8]: epoch at which block r landed in the local buffer
  int* chunk_counter;    // all-gather, local int[8]: copy CTAs finished per block (self-resetting)
  void* stage[8];        // reduce-scatter: staging buffer of every rank, [world][M/world, N] bf16
  void* rs_out;          // reduce-scatter: local result [M/world, N] bf16 (written by the fused reduce phase)
  int* tile_counter;     // reduce-scatter, local int[8]: epilogue-warp arrivals per destination (cleared at launch)
  // pair-tile engine (gemm_comm2.cu), reduce-scatter by pulling: `stage[r]` is then rank r's whole partial product
  // [M, N] in symmetric memory, `gathered` the local [world][M/world, N] buffer the peers' blocks are pulled into and
  // `pull_counter` a local int counting the CTAs that finished pulling (cleared at launch).  fuse_reduce: 1 = product,
  // pull and reduce in one launch; 0 = product + announcements only; 2 = pull + reduce only (the two halves let a test
  // run several ranks on one GPU without kernels waiting for one another).
  void* gathered;
  int* pull_counter;
  // pair-tile engine: shared-memory copy slots of the comm lane (1..3, each taken from the GEMM's operand stages);
  // 0 lets the launcher choose from the shape (transfer time against arithmetic time).
  int copy_slots = 0;
};
// The same two operations on the CTA-pair tile engine with in-kernel bulk-copy transfer (gemm_comm2.cu); they need
// M % (world * 256) == 0 (tp2_shape_ok) and are the ones the tensor-parallel layers use when the shape allows.
bool tp2_shape_ok(int M, int N, int K, int world);
int gemm_allgather2(const void* W, bool w_kmajor, void* Y, int M, int N, int K, long long ldy, const TpGemmParams& p,
                    int* status, cudaStream_t st);
int gemm_reducescatter2(const void* X, const void* W, bool w_kmajor, int M, int N, int K, const TpGemmParams& p,
                        int* status, cudaStream_t st);
// Y[M, N] = X_full[M, K] * op(W) where row block r of X_full is pulled from rank r inside the kernel.
// W is stored [N, K] (w_kmajor) or [K, N]; both contiguous.
int gemm_allgather(const void* W, bool w_kmajor, void* Y, int M, int N, int K, long long ldy, const TpGemmParams& p,
                   int* status, cudaStream_t st);
// Partial product X[M, K] * op(W) scattered to the owners of its row blocks and (fuse_reduce) summed there.
int gemm_reducescatter(const void* X, const void* W, bool w_kmajor, int M, int N, int K, const TpGemmParams& p,
                       int* status, cudaStream_t st);
// out[rows, N] = sum over the `world` slots of stage[world][rows, N].
int tp_reduce(const void* stage, void* out, long long rows, int N, int world, cudaStream_t st);

// ---- fp8 (gemm_fp8.cu).  q = x / *scale (saturating) as E4M3 or E5M2; `qt` (may be null) receives the transposed
// tensor [cols, rows]; `amax` (may be null, must start at 0) receives max|x|.
int fp8_quantize(const void* x, void* q, void* qt, const float* scale, float* amax, int rows, int cols, long long ldx,
                 bool e5m2, cudaStream_t st);
// D[M,N] bf16 = (A[M,K] . B[N,K]^T) * *scale_a * *scale_b (+ bias[N] bf16); A, B fp8, K a multiple of 16.
int gemm_fp8(const void* A, const void* B, void* D, const float* scale_a, const float* scale_b, const void* bias, int M,
             int N, int K, long long ldd, bool a_e5m2, bool b_e5m2, int* status, cudaStream_t st);

// ---- block-scaled fp8 (gemm_fp8_block.cu): E4M3 with one fp32 scale per 1 x 128 activation block / 128 x 128 weight block.
// sa_t is [cols / 128, rows] (block-major), sb is [ceil(rows / 128), cols / 128]; cols (= K) must be a multiple of 128.
int fp8_quantize_act_block(const void* x, void* q, float* sa_t, int rows, int cols, long long ldx, cudaStream_t st);
int fp8_quantize_weight_block(const void* w, void* q, float* sb, int rows, int cols, long long ldw, cudaStream_t st);
// D[M,N] bf16 = sum over K blocks of sa_t[kb, m] * sb[n / 128, kb] * (A[m, kb] . B[n, kb]) (+ bias[N] bf16).
int gemm_fp8_block(const void* A, const void* B, void* D, const float* sa_t, const float* sb, const void* bias, int M, int N, int K,
                   long long ldd, int* status, cudaStream_t st);

// ---- int8 (gemm_fp8.cu).  Symmetric per-row quantisation: scale[r] = max|x[r, :]| / 127, q = round(x / scale).
int int8_quantize_rows(const void* x, void* q, float* scale, int rows, int cols, long long ldx, cudaStream_t st);
// D[M,N] bf16 = (A[M,K] . B[N,K]^T in exact int32) * row_scale[m] * col_scale[n] (+ bias[N] bf16); K a multiple of 16.
int gemm_int8(const void* A, const void* B, void* D, const float* row_scale, const float* col_scale, const void* bias, int M,
              int N, int K, long long ldd, int* status, cudaStream_t st);

// ---- sampling (sampling.cu): one token per row of logits [rows, V] (bf16 or fp32, row stride ld elements).
// `work` fp32 [rows, V] receives the final (scaled, filtered, penalised) logits.  top_k / top_p / penalty / hist may be
// null.  hist int64 [rows, hist_len] with optional bool mask.  `all_greedy`: argmax of the raw logits for every row.
int sample_rows(const void* logits, bool is_bf16, long long ld, float* work, const float* temps, const int* top_k,
                const float* top_p, const float* penalty, const long long* hist, const bool* hist_mask, int hist_len,
                int rows, int V, bool all_greedy, unsigned long long seed, unsigned long long offset, long long* out_tok,
                float* out_logp, cudaStream_t st);

// ---- mixture of experts (moe.cu, gemm_grouped.cu)
int moe_router(const void* logits, void* probs, long long* idx, void* weights, int* counts, float* probsum, long long tokens,
               int E, int K, bool renorm, bool is_bf16, cudaStream_t st);
int moe_plan(const int* counts, int* offsets, int* tile_expert, int* cursors, int* total, int E, int max_tiles, cudaStream_t st);
int moe_permute(const void* x, const long long* idx, const int* counts, const int* offsets, int* cursors, void* sorted, int* slot_of,
                long long tokens, int K, int D, int E, bool is_bf16, cudaStream_t st);
int moe_combine(const void* y, const int* slot_of, const void* weights, void* out, long long tokens, int K, int D, bool is_bf16,
                cudaStream_t st);
int moe_combine_bwd(const void* dout, const void* y, const int* slot_of, const void* weights, void* dy, float* dw, long long tokens,
                    int K, int D, bool is_bf16, cudaStream_t st);
struct GroupedParams {
  const int* tile_expert;     // rows mode: expert of every 128-row tile of the sorted buffer (-1 = unused tile)
  const int* offsets;         // wgrad mode: padded segment offsets [E+1]
  int b_rows_per_expert;      // row stride between consecutive experts in the 2-D weight view
  int b_row_offset;           // first row of the wanted matrix inside an expert's block
  long long d_expert_stride;  // wgrad mode: elements between consecutive experts in the output
  int E;
};
// Expert-parallel extension of the rows mode.  Every rank owns E / world experts; the rows of its sorted buffer come
// from (gather) or go back to (scatter) the ranks whose tokens chose those experts.  row_peer[r] = rank << 24 | index
// names the peer row behind sorted row r (index = token * top_k + choice), -1 for padding rows.
//   gather : copy CTAs at the front of the grid pull the rows of the A operand from the peers' `src` buffers (bulk
//            copies through shared memory), zero the padding, and publish tile_flags[tile] = epoch; the GEMM CTAs poll a
//            tile's flag before its first TMA load.  The copy CTAs first (optionally) announce `announce_unit` to every
//            peer and wait for every peer's `wait_unit` flag: "your source rows and my table are complete".
//   scatter: the epilogue stores output row r into row `index` of the `dst` buffer of rank row_peer[r] >> 24; the last
//            CTA to finish publishes `signal_unit` to every peer.
struct EpRows {
  int world = 1, rank = 0;
  const int* row_peer = nullptr;
  const void* src[8] = {};     // gather: every rank's [*, K] bf16 rows; null = no gather
  int src_div = 1;             // gather: source row = index / src_div
  int* tile_flags = nullptr;   // gather: local int[R / 128]
  int n_copy_ctas = 0;
  void* dst[8] = {};           // scatter: every rank's [*, N] bf16 rows; null = no scatter
  int* done_counter = nullptr; // scatter: local int (self-resetting)
  void* flags[8] = {};         // flag array of every rank ([kind][8][max_units] int32)
  int announce_unit = -1, wait_unit = 0, signal_unit = 0, max_units = 8, epoch = 0;
  unsigned long long timeout_ns = 0;
};
int gemm_grouped_rows(const void* X, const void* W, void* Y, int R, int N, int K, long long ldx, long long w_rows, long long w_cols,
                      long long ldy, bool w_kmajor, const GroupedParams& g, int* status, cudaStream_t st,
                      const EpRows* ep = nullptr);
// Expert-parallel routing exchange (moe_ep.cu).  Step 1, every rank: blank the local row table, copy the local
// per-expert counts into row `rank` of every peer's counts table, publish `unit`.
int ep_push_counts(const int* counts_local, int E, void* const* counts_all, int* row_peer_local, int r_cap, void* const* flags,
                   int world, int rank, int unit, int max_units, int epoch, cudaStream_t st);
// Step 2, every rank: wait for all counts, lay out every rank's padded expert segments, write the local segment
// offsets [E / world + 1] / tile -> expert map [r_cap / 128] / row total, and enter this rank's (token, choice) pairs
// into the row tables of the ranks that own the chosen experts; publish `signal_unit`.
int ep_plan(const long long* idx, long long pairs, const int* counts_all_local, void* const* row_peer, int* offsets,
            int* tile_expert, int* total, int E, int r_cap, void* const* flags, int world, int rank, int wait_unit,
            int signal_unit, int max_units, int epoch, unsigned long long timeout_ns, int* status, cudaStream_t st);
int gemm_grouped_wgrad(const void* dY, const void* X, void* D, int R, int N, int K, long long lddy, long long ldx, long long ldd,
                       bool out_f32, bool accumulate, const GroupedParams& g, int* status, cudaStream_t st);

// Skinny GEMM for M <= 256 (gemm_skinny.cu): Y[M,N] bf16 = X[M,K] . W[N,K]^T with the weight as the MMA's M operand and
// K split over a thread-block cluster (reduction through distributed shared memory; no workspace).
int gemm_skinny_splits(int N, int K, int tok);
int gemm_skinny(const void* X, const void* W, void* Y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
                int* status, cudaStream_t st);

}  // namespace ab
