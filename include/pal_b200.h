/*
 * pal_b200 - C ABI of the B200 (sm_100a) paged-attention operator library.
 *
 * This is the boundary a host binding talks to.  It replaces the nanobind/MLX
 * primitive layer of Proxy Attention Lab (src/pal_core/bindings.cpp:40-222 and the
 * three Primitive::eval_gpu launchers behind it).  Every entry point takes plain
 * device pointers and sizes, launches asynchronously on the CUDA stream it is given
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), never
 * synchronises, never allocates device memory and owns nothing.
 *
 * Error convention: 0 = PAL_OK, negative = error; pal_last_error() returns a
 * thread-local message for the last failing call on this thread.  No exception or
 * abort crosses this boundary (the reference throws std::runtime_error /
 * std::invalid_argument instead: src/pal_core/src/paged_attention_decode_primitive.cpp:139-159).
 *
 * Cache layouts (shared with the reference, element type T is 2 bytes, x = 16/sizeof(T) = 8):
 *   K pool [P, Hkv, D/x, TPP, x]   src/pal_core/src/paged_attention_decode_primitive.cpp:384-397
 *   V pool [P, Hkv, D,   TPP]      src/pal_core/src/paged_attention_decode_primitive.cpp:373-382
 * page_table is [S, MP] 32-bit page ids (uint32 in the reference; int32 with the same bits is
 * accepted), lengths / positions are int32.
 */
#ifndef PAL_B200_H_
#define PAL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PAL_OK 0
#define PAL_ERR_BAD_ARG (-1)     /* null pointer, negative size, Hq % Hkv != 0 ...            */
#define PAL_ERR_UNSUPPORTED (-2) /* head_dim / tokens_per_page / dtype without an instantiation */
#define PAL_ERR_LAUNCH (-3)      /* CUDA reported an error at launch                            */
#define PAL_ERR_WORKSPACE (-4)   /* workspace missing or too small                              */
#define PAL_ERR_TIMEOUT (-5)     /* a bounded device-side wait gave up (read by pal_check_status) */

#define PAL_DTYPE_F16 0
#define PAL_DTYPE_BF16 1
/* OR this into the `dtype` argument of an attention entry point (decode, prefill, lse_combine) to have the
 * output written as float32 instead of the input type: the arithmetic is unchanged (16-bit inputs, fp32
 * accumulation), only the final rounding to 16 bits is left out.  No counterpart in the reference, whose
 * outputs always have the query dtype (src/pal_core/src/ops.cpp:93-94); it exists so that results can be
 * compared with an fp32 oracle free of output quantisation. */
#define PAL_OUT_F32 0x100

/* Value of partition_pages that selects the fused single-pass decode kernel, and the value
 * that lets the launcher choose (two-pass when the batch alone cannot fill the GPU). */
#define PAL_DECODE_SINGLE_PASS 0
#define PAL_DECODE_AUTO (-1)

const char* pal_last_error(void);
const char* pal_version(void);

/* ---- workspaces --------------------------------------------------------------------------- */
/* Every attention entry point takes a caller-owned device workspace (256-byte aligned; size from the
 * *_workspace_bytes functions).  Its first 256 bytes are a header: a work counter for the kernels' dynamic
 * scheduler and a status word.  The header must be zero before the first call that uses the workspace -
 * pal_workspace_init (a 256-byte cudaMemsetAsync on `stream`) does that, as does any other memset - and the
 * kernels leave it zeroed when they finish, so calls that follow one another on a stream need nothing in
 * between.  One workspace serves one call at a time: calls that may overlap on the GPU need one each.
 * No counterpart in the reference, where MLX's allocator provides temporaries
 * (src/pal_core/src/paged_attention_decode_primitive.cpp:163-175). */
int pal_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Every device-side wait in this library is bounded: when it has lasted `cycles` SM clock cycles the kernel
 * records PAL_ERR_TIMEOUT in the workspace status word and returns.  Sets the bound for the launches that
 * follow (process-wide; <= 0 restores the default of 4e9 cycles, about 2 s) and returns the previous one. */
int64_t pal_set_wait_limit_cycles(int64_t cycles);

/* Reads (with a blocking copy on `stream`) the status word the kernels of the last call that used
 * `workspace` left there: PAL_OK, or PAL_ERR_TIMEOUT when a bounded device-side wait gave up.  After a
 * timeout the header is zeroed again, so the workspace can be reused.  Optional; for tests and debugging. */
int pal_check_status(void* workspace, void* stream);

/* Launches one CTA that waits on a barrier nobody arrives at, bounded to `limit_cycles` (> 0): the wait
 * expires, the kernel records the timeout in `workspace` and returns normally.  Exists to test the
 * reporting path of the bounded waits (pal_check_status must then return PAL_ERR_TIMEOUT) without hanging
 * or faulting anything. */
int pal_selftest_bounded_wait(void* workspace, int64_t limit_cycles, void* stream);

/* ---- layout helpers ----------------------------------------------------------------------- */
/* src/pal_core/bindings.cpp:44-46 (get_k_cache_stripe_size) */
int pal_get_k_cache_stripe_size(int dtype);
/* src/pal_core/include/pal_core/constants.hpp:7-11 (get_optimal_page_size) */
int pal_get_optimal_page_size(void);
/* src/pal_core/src/paged_attention_decode_primitive.cpp:384-397 (get_k_cache_shape); writes 5 extents */
int pal_get_k_cache_shape(int64_t num_pages, int num_kv_heads, int head_dim, int tokens_per_page,
                          int dtype, int64_t shape_out[5]);
/* src/pal_core/src/paged_attention_decode_primitive.cpp:373-382 (get_v_cache_shape); writes 4 extents */
int pal_get_v_cache_shape(int64_t num_pages, int num_kv_heads, int head_dim, int tokens_per_page,
                          int dtype, int64_t shape_out[4]);

/* ---- fill_kv_pages ------------------------------------------------------------------------ */
/* Replaces FillKVPagesPrimitive::eval_gpu + fill_kv_pages_kernel
 * (src/pal_core/src/fill_kv_pages_primitive.cpp:70-170,
 *  src/pal_core/kernels/paged_attention/fill_kv_pages.h.metal:30-121).
 * Scatters new_keys/new_values [T, Hkv, D] into the pools IN PLACE (the reference copies
 * both pools first; a caller wanting that clones before the call).  Token t goes to page
 * page_table[query_to_seq_map[t], pos/TPP], slot pos%TPP with pos = write_positions[t].
 * Tokens whose page id is >= num_pages, whose sequence index is >= num_seqs or whose
 * logical block is >= max_pages_per_seq are skipped. */
int pal_fill_kv_pages(const void* new_keys, const void* new_values, void* k_pool, void* v_pool,
                      const void* page_table, const int32_t* write_positions,
                      const void* query_to_seq_map, int64_t num_tokens, int num_seqs,
                      int num_kv_heads, int head_dim, int tokens_per_page, int64_t num_pages,
                      int max_pages_per_seq, int dtype, void* stream);

/* Same scatter addressed by flat slot ids: slot_mapping[t] = page * TPP + slot_in_page (int64).
 * Tokens with a slot outside [0, num_pages*TPP) are skipped.  No counterpart in the reference
 * (which derives the slot in-kernel, fill_kv_pages.h.metal:64-72); this is the form serving
 * engines that keep a slot mapping already use. */
int pal_fill_kv_pages_slots(const void* new_keys, const void* new_values, void* k_pool,
                            void* v_pool, const int64_t* slot_mapping, int64_t num_tokens,
                            int num_kv_heads, int head_dim, int tokens_per_page,
                            int64_t num_pages, int dtype, void* stream);

/* ---- paged_attention_decode --------------------------------------------------------------- */
/* Bytes of device workspace pal_paged_attention_decode needs for this problem; depends on
 * partition_pages (see below).  Always >= 256. */
size_t pal_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                  int tokens_per_page, int max_pages_per_seq, int partition_pages);

/* The partition size PAL_DECODE_AUTO resolves to for this problem: 0 (single pass) when the batch alone gives
 * every resident CTA (two per SM) a (sequence, kv head) work item, otherwise the number of pages per partition
 * with the least modelled step time - the larger of the HBM time of all pages and the busiest CTA's own streaming
 * time, plus a fixed cost per work item and per partition merged: as few partitions as still keep most CTAs
 * busy in one wave, never below 16 pages.  The
 * reference switches to two passes by page-table width alone, with fixed 512-token chunks
 * (src/pal_core/src/paged_attention_decode_primitive.cpp:100-102). */
int pal_decode_auto_partition_pages(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                    int tokens_per_page, int max_pages_per_seq);

/* Replaces PagedAttentionDecodePrimitive::eval_gpu and its two kernels
 * (src/pal_core/src/paged_attention_decode_primitive.cpp:71-266,
 *  src/pal_core/kernels/paged_attention/decode/paged_attention_decode.h.metal:29-412,
 *  src/pal_core/kernels/paged_attention/decode/paged_reduce_decode.h.metal:27-129).
 * queries [>=S, Hq, D] (row s belongs to sequence s), out [S, Hq, D] in the query dtype (float32 with
 * dtype | PAL_OUT_F32).
 * A sequence of length <= 0 produces zeros.  scale <= 0 selects 1/sqrt(D).
 * partition_pages: PAL_DECODE_SINGLE_PASS (0) = one fused pass per (sequence, kv head);
 * n > 0 = split every sequence into partitions of n pages, write fp32 (m, l, acc) partials to
 * the workspace and merge them with the log-sum-exp combine kernel; PAL_DECODE_AUTO (-1) lets
 * the launcher choose.  Page ids are clamped to [0, num_pages) before use. */
int pal_paged_attention_decode(const void* queries, const void* k_pool, const void* v_pool,
                               const void* page_table, const int32_t* sequence_lengths, void* out,
                               int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                               int tokens_per_page, int64_t num_pages, int max_pages_per_seq,
                               float scale, int dtype, int partition_pages, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Same operation with the workspace taken from a PAL_STATIC_SCRATCH_BYTES array built into the library,
 * for hosts that own nothing but the tensors they were given (device memory fully committed to the page
 * pools, or a plugin interface with no way to request temporaries) and so cannot supply a workspace.
 * No counterpart in the reference, whose MLX allocator always hands its primitives scratch buffers.
 * The call allocates nothing.  It fails with PAL_ERR_WORKSPACE when the problem needs more than
 * PAL_STATIC_SCRATCH_BYTES (see pal_decode_workspace_bytes).  All calls on one GPU share the array and
 * it keeps the previous call's contents: calls that overlap on a GPU race, so serialise them.  The first
 * call on each device (this one or pal_static_scratch_init) loads the array's module - that is when the
 * device sets the 16 MiB aside, so it must come before the host commits its last free memory, and it fails
 * with PAL_ERR_WORKSPACE if the memory is not there - resolves the array's device address and zeroes its
 * header; make that call outside any stream capture.  pal_check_status_static reads the status word of the
 * built-in array (see pal_check_status). */
#define PAL_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
int pal_static_scratch_init(void);
int pal_check_status_static(void* stream);
int pal_paged_attention_decode_static(const void* queries, const void* k_pool, const void* v_pool,
                                      const void* page_table, const int32_t* sequence_lengths, void* out,
                                      int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                      int tokens_per_page, int64_t num_pages, int max_pages_per_seq,
                                      float scale, int dtype, int partition_pages, void* stream);

/* Fused "append + attend": the decode step a serving loop runs as fill_kv_pages for each sequence's newest
 * token followed by paged_attention_decode (src/proxy_attention_lab/ops.py:33-84 and :133-176 called back to
 * back; the reference has no fused form).  new_keys / new_values [S, Hkv, D] hold the K and V of the token at
 * position sequence_lengths[s] - 1 (the lengths already count it).  In one launch the kernel stores them into
 * page page_table[s, (L-1)/TPP], slot (L-1)%TPP of both pools - bit for bit what pal_fill_kv_pages would write -
 * and attends over all L tokens, taking the newest token from new_keys / new_values rather than from the pool.
 * Sequences of length <= 0, or whose last page lies beyond max_pages_per_seq, append nothing; a page id
 * >= num_pages is not written.  Everything else as pal_paged_attention_decode (same workspace rule). */
int pal_paged_attention_decode_append(const void* new_keys, const void* new_values, const void* queries,
                                      void* k_pool, void* v_pool, const void* page_table,
                                      const int32_t* sequence_lengths, void* out, int num_seqs,
                                      int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                                      int64_t num_pages, int max_pages_per_seq, float scale, int dtype,
                                      int partition_pages, void* workspace, size_t workspace_bytes,
                                      void* stream);

/* First half of the two-pass decode, for callers that merge partials themselves (for example
 * across GPUs that each hold a slice of every sequence's context).  Runs the split-KV pass over
 * the pages this pool holds and merges its own partitions, but does not normalise: writes
 * m_out [S, Hq] (max scaled score, natural-log units, -inf when the sequence is empty here),
 * l_out [S, Hq] (sum of exp(score - m)) and acc_out [S, Hq, D] (sum of exp(score - m) * v), fp32.
 * Shares the workspace rule of pal_paged_attention_decode with the same partition_pages (> 0). */
int pal_paged_attention_decode_partials(const void* queries, const void* k_pool, const void* v_pool,
                                        const void* page_table, const int32_t* sequence_lengths,
                                        float* m_out, float* l_out, float* acc_out, int num_seqs,
                                        int num_q_heads, int num_kv_heads, int head_dim,
                                        int tokens_per_page, int64_t num_pages,
                                        int max_pages_per_seq, float scale, int dtype,
                                        int partition_pages, void* workspace,
                                        size_t workspace_bytes, void* stream);

/* The same pass with the triple written as one buffer packed_out [S*Hq, D + 2] (fp32): per row D values of acc,
 * then m, then l - the form a single collective moves between GPUs.  Merge with pal_lse_combine_packed. */
int pal_paged_attention_decode_partials_packed(const void* queries, const void* k_pool, const void* v_pool,
                                               const void* page_table, const int32_t* sequence_lengths,
                                               float* packed_out, int num_seqs, int num_q_heads,
                                               int num_kv_heads, int head_dim, int tokens_per_page,
                                               int64_t num_pages, int max_pages_per_seq, float scale,
                                               int dtype, int partition_pages, void* workspace,
                                               size_t workspace_bytes, void* stream);

/* Log-sum-exp merge of num_parts partial triples per row (paged_reduce_decode.h.metal:79-128,
 * with fp32 un-normalised partials instead of the reference's 16-bit pre-normalised ones):
 * m, l are [num_parts, rows] and acc is [num_parts, rows, D] (part-major, the layout an
 * all-gather of per-GPU triples produces); out [rows, D] in `dtype`.  A row whose partials are
 * all empty becomes zeros. */
int pal_lse_combine(const float* m, const float* l, const float* acc, void* out, int num_parts,
                    int64_t rows, int head_dim, int dtype, void* stream);
/* The same merge reading packed [num_parts, rows, D + 2] (what an all-gather of the per-GPU packed_out buffers
 * of pal_paged_attention_decode_partials_packed produces), without unpacking. */
int pal_lse_combine_packed(const float* packed, void* out, int num_parts, int64_t rows, int head_dim,
                           int dtype, void* stream);

/* ---- context-sharded decode across GPUs --------------------------------------------------- */
/* For contexts so long that every GPU holds a slice of every sequence (page_table / sequence_lengths describe
 * this GPU's slice; a rank without tokens of a sequence passes length 0).  One call per GPU and step: the split-KV
 * pass over the local slice, then ONE kernel that merges the local partitions, stores the merged (acc, m, l) triple
 * of every row into every rank's exchange buffer with plain peer stores over NVLink, raises a flag, waits (bounded)
 * for the other ranks' triples and merges them into out [S, Hq, D] - every rank ends up with the full result.
 * No counterpart in the reference (single GPU).  The alternative without peer memory is
 * pal_paged_attention_decode_partials_packed + an all-gather (NCCL) + pal_lse_combine_packed.
 *
 * peer_bases: host array of world_size device addresses - rank r's exchange buffer as mapped into THIS process
 * (peer_bases[rank] is this GPU's own).  Each buffer has pal_exchange_bytes(world_size, rows_capacity, head_dim)
 * bytes, 256-byte aligned, peer-accessible, zeroed once on every rank before the first step (with a barrier
 * between the zeroing and the first call); rows_capacity >= S * Hq.  How the buffers are shared (CUDA IPC, a
 * symmetric-memory allocator, cuMem handles) is the caller's business.  All ranks must call once per step, in the
 * same order; steps may be captured in a CUDA graph (the step number lives in the buffer).  A wait that expires
 * leaves PAL_ERR_TIMEOUT in the workspace status word and the exchange buffers unusable until zeroed again. */
size_t pal_exchange_bytes(int world_size, int64_t rows_capacity, int head_dim);
int pal_paged_attention_decode_ctx_exchange(const void* queries, const void* k_pool, const void* v_pool,
                                            const void* page_table, const int32_t* sequence_lengths, void* out,
                                            int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                            int tokens_per_page, int64_t num_pages, int max_pages_per_seq,
                                            float scale, int dtype, int partition_pages, void* workspace,
                                            size_t workspace_bytes, const void* const* peer_bases,
                                            int world_size, int rank, int64_t rows_capacity, void* stream);

/* ---- paged_attention_prefill -------------------------------------------------------------- */
/* Bytes of workspace a prefill call of this shape can use (tokens_per_seq: the uniform count, or the longest sequence's
 * count for the ragged form): the 256-byte header, plus - for batches too small to give every SM a CTA - room for the
 * fp32 partial results of a launch that is cut along the history (at most 32 MB).  A call given only the header still
 * works; it runs uncut. */
size_t pal_prefill_workspace_bytes(int num_seqs, int tokens_per_seq, int num_q_heads,
                                   int num_kv_heads, int head_dim);

/* Replaces PagedAttentionPrefillPrimitive::eval_gpu and pal_paged_attention_prefill
 * (src/pal_core/src/paged_attention_prefill_primitive.cpp:63-167,
 *  src/pal_core/kernels/paged_attention/prefill/paged_attention_prefill.h.metal:28-389).
 * q_prompt [S*N, Hq, D], k_prompt / v_prompt [S*N, Hkv, D] dense (sequence-major, then token);
 * history_lens[s] tokens of history are read from the pages; out [S*N*Hq, D], row
 * (s*N + i)*Hq + h.  Query i sees all history tokens and new tokens 0..i.
 * dtype may carry PAL_OUT_F32 (float32 output).
 * impl: 0 = let the launcher choose (a tcgen05 kernel for every supported shape),
 * 1 = mma.sync kernel (every supported shape),
 * 2 = tcgen05/TMEM kernel (head_dim 32 / 64 / 80 / 96 / 128 / 256 with tokens_per_page 16 / 32: every supported shape),
 *     in the form the launcher prefers for the shape,
 * 3 = tcgen05, one accumulator tile per CTA with S double-buffered,
 * 4 = tcgen05, two CTAs per MMA (cta_group::2; head_dim 256, and head_dim 128 with an even number of query heads per
 *     kv head; PAL_ERR_UNSUPPORTED otherwise; what 0 and 2 choose for head_dim 256). */
int pal_paged_attention_prefill(const void* q_prompt, const void* k_prompt, const void* v_prompt,
                                const void* k_pool, const void* v_pool, const void* page_table,
                                const int32_t* history_lens, void* out, int num_seqs,
                                int tokens_per_seq, int num_q_heads, int num_kv_heads, int head_dim,
                                int tokens_per_page, int64_t num_pages, int max_pages_per_seq,
                                float scale, int dtype, int impl, void* workspace,
                                size_t workspace_bytes, void* stream);

/* Ragged form of pal_paged_attention_prefill: sequence s brings cu_seqlens[s+1] - cu_seqlens[s] new tokens (any
 * count, zero included), stored back to back: q_prompt [total_tokens, Hq, D], k_prompt / v_prompt
 * [total_tokens, Hkv, D], out [total_tokens*Hq, D]; cu_seqlens is a device array of num_seqs + 1 int32 row offsets
 * with cu_seqlens[0] = 0 and cu_seqlens[num_seqs] = total_tokens.  max_new_tokens is the largest count (it sizes
 * the grid; a smaller value than the truth leaves the tail of long sequences unwritten).  A batch that mixes prefill
 * chunks with single-token decode steps is the case count = 1.  No counterpart in the reference, which derives one
 * uniform count as q.shape(0) / num_sequences (src/pal_core/src/paged_attention_prefill_primitive.cpp:115-116).
 * With equal counts the result is bit-identical to pal_paged_attention_prefill. */
int pal_paged_attention_prefill_ragged(const void* q_prompt, const void* k_prompt, const void* v_prompt,
                                       const void* k_pool, const void* v_pool, const void* page_table,
                                       const int32_t* history_lens, const int32_t* cu_seqlens, void* out,
                                       int num_seqs, int64_t total_tokens, int max_new_tokens, int num_q_heads,
                                       int num_kv_heads, int head_dim, int tokens_per_page, int64_t num_pages,
                                       int max_pages_per_seq, float scale, int dtype, int impl, void* workspace,
                                       size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PAL_B200_H_ */
