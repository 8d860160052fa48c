// C entry point of the paged decode attention for callers that must not allocate device memory.
//
// This function has no counterpart in the reference project.  It exists for hosts that embed this library where
// cudaMalloc is off limits at call time: a serving loop whose memory pool already owns every byte of the GPU,
// a plugin loaded into a process that forbids allocation after start-up, or code running between the begin and
// end of a section in which the CUDA allocator may not be entered.  The regular entry (`ab::paged_decode`, and the
// torch op built on it) asks its caller for three scratch tensors; this one carries its scratch inside the
// library image instead, in a file-scope `__device__` array of fixed size.
//
// Limits (checked, with an error string, before anything is launched):
//   batch * n_q_heads * head_dim            <= ASTRAI_B200_NOALLOC_MAX_QELEMS  (131072: e.g. 32 requests x 32 heads x 128)
//   batch * n_q_heads and batch * n_kv_heads <= ASTRAI_B200_NOALLOC_MAX_HEADS  (4096)
//   KV splits are capped at ASTRAI_B200_NOALLOC_MAX_SPLITS (8)
// The array takes about 4.3 MB on every GPU on which the library is loaded, until the process exits.
//
// Behaviour to know about:
//   * The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress, with
//     that device current).  Make that first call outside of any stream capture.
//   * All calls share the one array.  Two calls whose kernels can overlap on the GPU (different streams without
//     an ordering between them) race on it; order them.
//   * The split counters are cleared on the given stream at the start of every call; partial results of the
//     previous call are simply overwritten.
//   * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
//
// Preconditions the function cannot check from raw pointers (the caller owns them):
//   * every req_pool_indices[i] names an existing row of req_to_token (a negative entry makes that request attend to
//     nothing; an entry past the last row reads memory that is not the table);
//   * seq_lens[i] <= max_ctx is enforced on the device by cutting longer lengths down to max_ctx, and slot numbers
//     outside [0, n_slots) found in the table are skipped, so neither can read outside the buffers.
#pragma once

#define ASTRAI_B200_NOALLOC_MAX_SPLITS 8
#define ASTRAI_B200_NOALLOC_MAX_QELEMS 131072
#define ASTRAI_B200_NOALLOC_MAX_HEADS 4096

#ifdef __cplusplus
extern "C" {
#endif

// Decode attention of one new token per request over a slot-addressed bf16 KV pool.
//   q, out           : [batch, n_q_heads, head_dim] bf16, contiguous, device memory
//   k_buf, v_buf     : [n_slots, n_kv_heads, head_dim] bf16
//   req_to_token     : [rows, max_ctx] int32 slot table; req_pool_indices [batch] int32 picks each request's row
//   seq_lens         : [batch] int64 number of cached tokens per request; max_len = their maximum (host value,
//                      only used to pick the number of KV splits)
//   stream           : a cudaStream_t (0 for the legacy default stream)
// Returns 0 on success, a negative code otherwise; astrai_b200_noalloc_error() then describes the failure.
int astrai_b200_paged_decode_noalloc(const void* q, const void* k_buf, const void* v_buf, const int* req_to_token,
                                     const int* req_pool_indices, const long long* seq_lens, void* out, int batch,
                                     int n_q_heads, int n_kv_heads, int head_dim, int max_ctx, long long n_slots,
                                     long long max_len, float scale, void* stream);

// Message of the last failure on the calling thread ("" if none).
const char* astrai_b200_noalloc_error(void);

#ifdef __cplusplus
}
#endif
