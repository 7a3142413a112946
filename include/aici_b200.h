/*
 * aici_b200 -- C ABI of the B200 (sm_100a) attention path for rLLM.
 *
 * These entry points are what rllm/tch-cuda/src/lib.rs would bind in place of the
 * `*_C(C_tensor*...)` externs (lib.rs:29-47, 106-190).  They take raw device pointers,
 * explicit sizes and element strides and a CUDA stream; no libtorch type crosses the
 * boundary.  Every function that can fail returns the reference's error convention
 * (lib.rs:12-27, kernels/vllm_bindings.cpp:7-13): NULL on success, otherwise a
 * malloc()-allocated, NUL-terminated message that the caller releases with free().
 *
 * Supported shapes: bf16 (AICI_DTYPE_BF16), head_size 128, block_size 16,
 * num_heads / num_kv_heads in {1, 2, 4, 8}.  Anything else returns an error string; there
 * is no fallback path.
 *
 * KV-cache layout (rllm-cuda/src/llm/paged/cache_engine.rs:81-108), x = 16 / sizeof(T) = 8:
 *   key_cache   [num_blocks, num_kv_heads, head_size / x, block_size, x]
 *   value_cache [num_blocks, num_kv_heads, head_size, block_size]
 *
 * Current device: every entry point launches on the CURRENT CUDA device of the calling thread, and
 * the tensors it is given must live there (outputs of other ranks in the `*_peers` calls excepted).
 * The reference's wrappers inherit this from libtorch's device guard; a caller of this C ABI makes
 * the tensors' GPU current itself (cudaSetDevice).  A mismatch is refused with an error string.
 *
 * Threads: the entry points are re-entrant.  The library keeps no mutable state a caller can
 * observe, apart from the device status word below, per-device one-time set-up done under a lock,
 * and a mutex-guarded table of encoded tensor maps keyed by (address, shape, strides).
 */
#ifndef AICI_B200_H_
#define AICI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *aici_stream_t; /* cudaStream_t */

enum { AICI_DTYPE_BF16 = 0, AICI_DTYPE_F16 = 1, AICI_DTYPE_F32 = 2 };

/* Sticky device-side status bits, read with aici_last_status(). */
enum {
  AICI_STATUS_OK = 0,
  AICI_STATUS_BAD_BLOCK = 1,   /* a block-table entry was outside [0, num_blocks)        */
  AICI_STATUS_BAD_SLOT = 2,    /* a slot index was outside the cache                      */
  AICI_STATUS_WAIT_TIMEOUT = 4, /* a bounded wait on a shared-memory barrier gave up      */
  AICI_STATUS_PEER_TIMEOUT = 8  /* a peer GPU did not reach a barrier within its bounded wait */
};

/* Library version string (static storage). */
const char *aici_version(void);

/* Reads and clears the sticky status word of the current device (synchronises the
 * device).  Kernels never trap: an out-of-range block or slot is skipped and recorded, and a wait
 * that ran out is recorded and abandoned, so the result of THAT launch is incomplete while later
 * launches run normally (no kernel reads the sticky bits).  A serving loop therefore polls this word
 * where it synchronises anyway (once per step, or every few steps) and treats a non-zero value as
 * the failure of the steps since the last poll. */
char *aici_last_status(int *status_out);

/* ---- KV-cache operations (bit-exact) ------------------------------------------------ */

/* Replaces reshape_and_cache_C (lib.rs:168-174; kernels/vllm/cache_kernels.cu:168-253).
 * key/value [num_tokens, num_kv_heads, head_size] with token strides in elements.
 * slot_mapping holds num_tokens entries, int64 when slot_is_int64 != 0 (what the Rust
 * wrapper passes after its cast, lib.rs:199-200) or int32 (what rLLM builds,
 * paged/batch_info.rs:203,271).  Negative slots are skipped. */
char *aici_reshape_and_cache(const void *key, const void *value, void *key_cache,
                             void *value_cache, const void *slot_mapping, int slot_is_int64,
                             int num_tokens, int num_kv_heads, int head_size, int block_size,
                             int64_t num_blocks, int64_t key_stride, int64_t value_stride,
                             int dtype, aici_stream_t stream);

/* Replaces gather_cached_kv_C (lib.rs:176-182; cache_kernels.cu:301-413): the inverse of
 * the above with int32 slots. */
char *aici_gather_cached_kv(void *key, void *value, const void *key_cache,
                            const void *value_cache, const int32_t *slot_mapping,
                            int num_tokens, int num_kv_heads, int head_size, int block_size,
                            int64_t num_blocks, int64_t key_stride, int64_t value_stride,
                            int dtype, aici_stream_t stream);

/* Replaces copy_blocks_2_C (lib.rs:184-189; cache_kernels.cu:141-163, kernel :55-81).
 * key_cache_ptrs / value_cache_ptrs: device arrays of num_layers base addresses;
 * block_mapping: device array of 2*num_pairs int64 (src, dst, src, dst, ...);
 * numel_per_block = num_kv_heads * head_size * block_size. */
char *aici_copy_blocks(const int64_t *key_cache_ptrs, const int64_t *value_cache_ptrs,
                       const int64_t *block_mapping, int num_layers, int num_pairs,
                       int64_t numel_per_block, int64_t num_blocks, int dtype,
                       aici_stream_t stream);

/* Same operation with all three arrays in HOST memory: the layer addresses and pairs
 * travel as kernel arguments, so the three blocking host-to-device uploads the Rust
 * wrapper makes per call (lib.rs:316-318) disappear.  Replaces tch_cuda::copy_blocks
 * (lib.rs:276-331) as a whole. */
char *aici_copy_blocks_host(const int64_t *key_cache_ptrs_host,
                            const int64_t *value_cache_ptrs_host,
                            const int64_t *block_mapping_host, int num_layers, int num_pairs,
                            int64_t numel_per_block, int64_t num_blocks, int dtype,
                            aici_stream_t stream);

/* Rotary embedding fused with the cache write: rotary_embedding_C (lib.rs:139-146;
 * kernels/vllm/pos_encoding_kernels.cu:40-128) followed by reshape_and_cache_C, as rLLM issues
 * them back to back (rllm-cuda/src/llm/mod.rs:107-114, 158-164), in one pass.  query
 * [num_tokens, num_heads, head_size] and key [num_tokens, num_kv_heads, head_size] are rotated in
 * place (NeoX pairing, bf16 arithmetic as in the reference kernel); the rotated key and `value` are
 * written to the paged cache at slot_mapping.  positions int64 [num_tokens]; cos_sin_cache
 * [max_position, rot_dim] = [cos | sin].  Requires rot_dim == head_size == 128 and is_neox != 0. */
char *aici_rotary_reshape_and_cache(const int64_t *positions, void *query, void *key,
                                    const void *value, const void *cos_sin_cache, void *key_cache,
                                    void *value_cache, const void *slot_mapping, int slot_is_int64,
                                    int num_tokens, int num_heads, int num_kv_heads, int head_size,
                                    int rot_dim, int is_neox, int64_t max_position, int block_size,
                                    int64_t num_blocks, int64_t query_stride, int64_t key_stride,
                                    int64_t value_stride, int dtype, aici_stream_t stream);

/* ---- decode attention over the paged cache ----------------------------------------- */

/* Bytes of caller-owned scratch aici_paged_attention_v1 needs for these sizes: about 520 bytes
 * per query head of a group and (warp of the grid + sequence x kv head); for batches above 2048
 * sequences per (sequence, head, chunk).  Depends on its arguments and the device only. */
size_t aici_paged_attention_workspace_bytes(int num_seqs, int num_heads, int num_kv_heads,
                                            int max_context_len);

/* Replaces paged_attention_v1_C (lib.rs:108-120; vllm_bindings.cpp:17-29;
 * kernels/vllm/attention/attention_kernels.cu:571-700).  out/query
 * [num_seqs, num_heads, head_size] (q_stride = query row stride in elements; out is
 * contiguous); block_tables int32 [num_seqs, max_num_blocks_per_seq]; context_lens int32
 * [num_seqs]; kv_block_stride / kv_head_stride in elements.  alibi_slopes must be NULL
 * (rLLM never passes one, rllm-cuda/src/llm/mod.rs:310).  Rows of the batch that more than one
 * warp worked on are combined by a second kernel; `workspace` holds the traversal's bookkeeping
 * and the fp32 partial results, needs no initialisation, and must be at least
 * aici_paged_attention_workspace_bytes() large and 256-byte aligned. */
char *aici_paged_attention_v1(void *out, const void *query, const void *key_cache,
                              const void *value_cache, int num_kv_heads, float scale,
                              const int32_t *block_tables, const int32_t *context_lens,
                              int block_size, int max_context_len, const float *alibi_slopes,
                              int num_seqs, int num_heads, int head_size,
                              int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                              int64_t kv_block_stride, int64_t kv_head_stride, void *workspace,
                              size_t workspace_bytes, int dtype, aici_stream_t stream);

/* Test and benchmark hook (no counterpart in the reference): aici_paged_attention_v1 through the
 * other traversal -- every sequence cut into chunks of chunk_tokens tokens (a multiple of 16 up to
 * 512; 0 = the library's own choice), dealt out round-robin -- so that the two can be compared.
 * The chunk size is an argument of the call; its workspace size comes from
 * aici_paged_attention_chunked_workspace_bytes with the same chunk_tokens. */
size_t aici_paged_attention_chunked_workspace_bytes(int num_seqs, int num_heads, int num_kv_heads,
                                                    int max_context_len, int chunk_tokens);
char *aici_paged_attention_v1_chunked(void *out, const void *query, const void *key_cache,
                                      const void *value_cache, int num_kv_heads, float scale,
                                      const int32_t *block_tables, const int32_t *context_lens,
                                      int block_size, int max_context_len, const float *alibi_slopes,
                                      int num_seqs, int num_heads, int head_size,
                                      int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                                      int64_t kv_block_stride, int64_t kv_head_stride, void *workspace,
                                      size_t workspace_bytes, int chunk_tokens, int dtype,
                                      aici_stream_t stream);

/* Replaces paged_attention_v2_C (lib.rs:122-137; vllm_bindings.cpp:31-45;
 * attention_kernels.cu:729-874).  Partition size 512 as in the reference (:733);
 * exp_sums / max_logits fp32 [num_seqs, num_heads, P], tmp_out T
 * [num_seqs, num_heads, P, head_size], P = ceil(max_context_len / 512), filled with the
 * reference's meaning (partition max logit, partition exp sum, partition-normalised
 * output) for every partition that holds at least one token. */
char *aici_paged_attention_v2(void *out, float *exp_sums, float *max_logits, void *tmp_out,
                              const void *query, const void *key_cache,
                              const void *value_cache, int num_kv_heads, float scale,
                              const int32_t *block_tables, const int32_t *context_lens,
                              int block_size, int max_context_len, const float *alibi_slopes,
                              int num_seqs, int num_heads, int head_size,
                              int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                              int64_t kv_block_stride, int64_t kv_head_stride, int dtype,
                              aici_stream_t stream);

/* Same operation and arguments as aici_paged_attention_v1 without the workspace: the scratch
 * lives in a 32 MiB array built into the library (present on every GPU that loads it).  This
 * entry point has no counterpart in the reference.  It is meant for callers that must not
 * allocate device memory at call time -- a serving loop that gave all spare memory to the KV
 * pool, or a binding without a device allocator -- and it calls no allocation routine itself.
 * Batches whose workspace (aici_paged_attention_workspace_bytes) exceeds 32 MiB are refused with
 * an error string (argument errors are reported first).  All calls on one device share the array:
 * calls that overlap on the GPU race, so keep them on one stream.  The first call on a device looks up the array's address; make it
 * outside any stream capture. */
char *aici_paged_attention_v1_static(void *out, const void *query, const void *key_cache,
                                     const void *value_cache, int num_kv_heads, float scale,
                                     const int32_t *block_tables, const int32_t *context_lens,
                                     int block_size, int max_context_len,
                                     const float *alibi_slopes, int num_seqs, int num_heads,
                                     int head_size, int max_num_blocks_per_seq, int64_t num_blocks,
                                     int64_t q_stride, int64_t kv_block_stride,
                                     int64_t kv_head_stride, int dtype, aici_stream_t stream);

/* ---- variable-length causal prefill attention --------------------------------------- */

/* Replaces mha_varlen_fwd_C (lib.rs:29-47; kernels/flash_attn/flash_api.cpp:622-655,
 * 447-618).  q/out [total_q, num_heads, head_size], k/v [total_k, num_heads_k, head_size];
 * token and head strides in elements, last dimension contiguous; cu_seqlens_{q,k} int32
 * [batch + 1] on the device.  The causal mask is aligned to the bottom-right corner of each
 * sequence's (len_q x len_k) score matrix.  The caller allocates `out` (the reference
 * allocated it, flash_api.cpp:542). */
char *aici_mha_varlen_fwd(void *out, const void *q, const void *k, const void *v,
                          const int32_t *cu_seqlens_q, const int32_t *cu_seqlens_k, int batch,
                          int total_q, int total_k, int num_heads, int num_heads_k,
                          int head_size, int max_seqlen_q, int max_seqlen_k,
                          int64_t q_tok_stride, int64_t q_head_stride, int64_t k_tok_stride,
                          int64_t k_head_stride, int64_t v_tok_stride, int64_t v_head_stride,
                          int64_t o_tok_stride, int64_t o_head_stride, float softmax_scale,
                          int is_causal, int dtype, aici_stream_t stream);

/* Test and benchmark hook (no counterpart in the reference): aici_mha_varlen_fwd with the kernel
 * shape given by the caller instead of chosen by sequence length.  shape 0 = automatic (what
 * aici_mha_varlen_fwd does: 1 up to 1024 keys, 2 above), 1 = one query tile per CTA, two CTAs per
 * SM, 2 = two query tiles per CTA sharing their key/value tiles, 3 = shape 2 on pairs of CTAs whose
 * MMAs span two SMs (tcgen05 cta_group::2; needs num_heads / num_heads_k to be a multiple of 4). */
char *aici_mha_varlen_fwd_shape(void *out, const void *q, const void *k, const void *v,
                                const int32_t *cu_seqlens_q, const int32_t *cu_seqlens_k, int batch,
                                int total_q, int total_k, int num_heads, int num_heads_k, int head_size,
                                int max_seqlen_q, int max_seqlen_k, int64_t q_tok_stride,
                                int64_t q_head_stride, int64_t k_tok_stride, int64_t k_head_stride,
                                int64_t v_tok_stride, int64_t v_head_stride, int64_t o_tok_stride,
                                int64_t o_head_stride, float softmax_scale, int is_causal, int shape,
                                int dtype, aici_stream_t stream);

/* ---- multi-GPU: attention whose epilogue is the head-output gather -------------------------
 * The reference has no multi-GPU code; its only hook is the per-rank kv-head count
 * (rllm-cuda/src/llm/config.rs:49-51).  With kv heads sharded over the GPUs of one box every rank
 * needs all heads of the attention output afterwards.  These two entry points write each finished
 * output row / tile straight into the output buffer of EVERY rank (outs[0..world), peer-mapped
 * device pointers, this rank's own included; each buffer [rows, total_heads, 128]) at head index
 * head0 + h, so no collective follows: the ranks only synchronise (a barrier) before reading.
 * A peer may start the next call while this rank still reads the buffer, so a caller either
 * alternates between two output buffers or places a second barrier after the readers.
 * Everything else is as in aici_paged_attention_v1 / aici_mha_varlen_fwd. */
char *aici_paged_attention_v1_peers(void *const *outs, int world, int total_heads, int head0,
                                    const void *query, const void *key_cache,
                                    const void *value_cache, int num_kv_heads, float scale,
                                    const int32_t *block_tables, const int32_t *context_lens,
                                    int block_size, int max_context_len, int num_seqs,
                                    int num_heads, int head_size, int max_num_blocks_per_seq,
                                    int64_t num_blocks, int64_t q_stride, int64_t kv_block_stride,
                                    int64_t kv_head_stride, void *workspace, size_t workspace_bytes,
                                    int dtype, aici_stream_t stream);

char *aici_mha_varlen_fwd_peers(void *const *outs, int world, int head0, const void *q,
                                const void *k, const void *v, const int32_t *cu_seqlens_q,
                                const int32_t *cu_seqlens_k, int batch, int total_q, int total_k,
                                int num_heads, int num_heads_k, int head_size, int max_seqlen_q,
                                int max_seqlen_k, int64_t q_tok_stride, int64_t q_head_stride,
                                int64_t k_tok_stride, int64_t k_head_stride, int64_t v_tok_stride,
                                int64_t v_head_stride, int64_t o_tok_stride, int64_t o_head_stride,
                                float softmax_scale, int is_causal, int dtype, aici_stream_t stream);

/* Barrier between the ranks that share peer-mapped buffers (no counterpart in the reference).
 * flag_ptrs[p] = rank p's array of 32 uint32 slots (128 bytes) in peer-mapped memory, all zero
 * before the first call; every rank must call it the same number of times (the epoch is a counter
 * kept in the array, so a captured launch can be replayed).  Enqueued on `stream`: work queued after it starts
 * once every rank's earlier work on its own stream has finished.  The wait is bounded (about a
 * second), then AICI_STATUS_PEER_TIMEOUT is recorded and the kernel returns. */
char *aici_peer_barrier(void *const *flag_ptrs, int world, int rank, aici_stream_t stream);

/* aici_paged_attention_v1_peers with that barrier folded into its last kernel: when the call's
 * kernels have finished, every rank's buffer holds all heads, and no barrier launch follows (one
 * launch less per decode step).  flag_ptrs as for aici_peer_barrier; the two may be mixed on the
 * same arrays as long as all ranks make the same sequence of calls (this one counts arrivals in
 * slots 16-23 and its calls in slot 10; the barrier kernel uses slots 0-8).  Every CTA of the last
 * kernel reports to every rank once its rows are stored there, and one CTA waits until every rank
 * has reported in full: bounded, AICI_STATUS_PEER_TIMEOUT as above. */
char *aici_paged_attention_v1_peers_barrier(void *const *outs, void *const *flag_ptrs, int world,
                                            int rank, int total_heads, int head0, const void *query,
                                            const void *key_cache, const void *value_cache,
                                            int num_kv_heads, float scale, const int32_t *block_tables,
                                            const int32_t *context_lens, int block_size,
                                            int max_context_len, int num_seqs, int num_heads,
                                            int head_size, int max_num_blocks_per_seq,
                                            int64_t num_blocks, int64_t q_stride,
                                            int64_t kv_block_stride, int64_t kv_head_stride,
                                            void *workspace, size_t workspace_bytes, int dtype,
                                            aici_stream_t stream);

/* One decode step of one layer in one call: aici_reshape_and_cache of the step's new tokens (token i
 * is the newest token of sequence i: key/value [num_seqs, num_kv_heads, 128], slot_mapping[i] the
 * cache slot of position context_lens[i] - 1) followed by aici_paged_attention_v1 -- the two crate
 * calls rLLM makes back to back per layer (rllm-cuda/src/llm/mod.rs:132-166, 280-316).  The cache
 * write has no launch of its own here: the warp of the decode kernel that reaches the last tile of a
 * (sequence, kv head) row takes the new token from new_key / new_value, uses it, and writes it to
 * the cache.  A slot that is not the sequence's last position is recorded as AICI_STATUS_BAD_SLOT
 * and not written; a negative slot means "no new token" as in aici_reshape_and_cache.  At most 2048
 * sequences.  world == 1: outs[0] is the output [num_seqs, num_heads, 128], flag_ptrs may be NULL,
 * total_heads = num_heads, head0 = 0.  world > 1: as aici_paged_attention_v1_peers_barrier. */
char *aici_decode_step(void *const *outs, void *const *flag_ptrs, int world, int rank, int total_heads,
                       int head0, const void *new_key, const void *new_value, const void *slot_mapping,
                       int slot_is_int64, int64_t key_stride, int64_t value_stride, const void *query,
                       void *key_cache, void *value_cache, int num_kv_heads, float scale,
                       const int32_t *block_tables, const int32_t *context_lens, int block_size,
                       int max_context_len, int num_seqs, int num_heads, int head_size,
                       int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_stride,
                       int64_t kv_block_stride, int64_t kv_head_stride, void *workspace,
                       size_t workspace_bytes, int dtype, aici_stream_t stream);

/* Peer-mapped device memory without libtorch or NCCL (no counterpart in the reference, which is
 * single-GPU; the hook this serves is the per-rank kv-head count of
 * rllm-cuda/src/llm/config.rs:30-36, 49-51).  One process per GPU:
 *   owner : aici_peer_alloc(bytes, &ptr, handle)  -- zero-filled device memory + a 128-byte handle
 *   caller: moves the handle bytes to the other processes over any channel it has
 *   peers : aici_peer_open(handle, &ptr)          -- maps the owner's buffer into this process
 * The memory is a CUDA virtual-memory allocation (2 MB pages) shared through a file descriptor that
 * the peer duplicates with pidfd_getfd; where that is not possible, cudaMalloc with a CUDA IPC
 * handle.  The handle says which; processes must share a PID namespace (one container).
 * The pointers go into outs[] / flag_ptrs[] above (index = owner's rank; a rank's own buffer is the
 * pointer aici_peer_alloc gave it).  Tear-down: every peer aici_peer_close()s its mappings, the
 * processes meet (the caller's own barrier), then each owner aici_peer_free()s.  These four calls
 * allocate or map memory and synchronise the device: set-up time only, never inside a step. */
#define AICI_PEER_HANDLE_BYTES 128
char *aici_peer_alloc(size_t bytes, void **ptr_out, void *handle_out);
char *aici_peer_open(const void *handle, void **ptr_out);
char *aici_peer_close(void *ptr);
char *aici_peer_free(void *ptr);

/* The head-output gather as a call of its own, for attention results computed without the fused
 * epilogue: local [rows, num_heads, 128] (row stride in elements) is stored at head index
 * head0 + h of every rank's [rows, total_heads, 128] buffer (outs[0..world), peer-mapped, own
 * included) with 16-byte stores over NVLink.  Follow it with aici_peer_barrier before reading. */
char *aici_gather_heads(void *const *outs, int world, int total_heads, int head0, const void *local,
                        int64_t rows, int num_heads, int head_size, int64_t local_row_stride,
                        int dtype, aici_stream_t stream);

/* Variable-length causal prefill that reads keys and values straight from the paged cache.
 * Replaces the sequence gather_cached_kv -> repeat_kv -> flash_attn_varlen of
 * compute_varlen_attn (rllm-cuda/src/llm/mod.rs:168-278; kernels/vllm/cache_kernels.cu:301-413):
 * no packed copy of the context is made and no head is replicated.  q/out as in
 * aici_mha_varlen_fwd; sequence i attends to its first context_lens[i] tokens, found through row i
 * of block_tables (int32 [batch, max_num_blocks_per_seq]; logical token t lives in block
 * table[t / 16] at offset t % 16, as rLLM allocates, paged/blocks.rs:122-127).  The causal mask is
 * bottom-right aligned, so a chunk of new tokens after an already cached prefix is
 * len_q < context_len.  Cache slots past context_lens[i] may hold anything. */
char *aici_mha_varlen_paged_fwd(void *out, const void *q, const void *key_cache,
                                const void *value_cache, const int32_t *cu_seqlens_q,
                                const int32_t *context_lens, const int32_t *block_tables, int batch,
                                int total_q, int num_heads, int num_kv_heads, int head_size,
                                int block_size, int max_seqlen_q, int max_context_len,
                                int max_num_blocks_per_seq, int64_t num_blocks, int64_t q_tok_stride,
                                int64_t q_head_stride, int64_t o_tok_stride, int64_t o_head_stride,
                                int64_t kv_block_stride, int64_t kv_head_stride, float softmax_scale,
                                int is_causal, int dtype, aici_stream_t stream);

/* ---- swap_blocks ---------------------------------------------------------------------------
 * Replaces swap_blocks (rllm/tch-cuda/kernels/vllm/cache_kernels.cu:12-50), which rLLM's
 * CacheEngine::swap calls per layer for K and for V (rllm-cuda/src/llm/paged/cache_engine.rs:139-149)
 * and which issues one cudaMemcpyAsync per block.  dst[block d] = src[block s] for every (s, d) of
 * block_mapping_host (host array of 2*num_pairs int64).  src and dst are the bases of two caches of
 * block_bytes-sized blocks; where each lives is read from the pointer itself: device <-> device on
 * one GPU, device <-> page-locked host (one kernel launch moves all blocks over PCIe), or
 * device <-> pageable host (copy engine, one transfer per run of consecutive blocks).  Host <-> host
 * is refused ("Invalid device combination"), two different GPUs too, as in the reference.
 * Stream-ordered; a host-side cache must stay untouched until the stream reaches the call. */
char *aici_swap_blocks(const void *src, void *dst, const int64_t *block_mapping_host, int num_pairs,
                       int64_t block_bytes, int64_t src_num_blocks, int64_t dst_num_blocks,
                       aici_stream_t stream);

/* ---- BatchInfo staging ---------------------------------------------------------------------
 * Replaces BatchInfoBuilder::finish (rllm-cuda/src/llm/paged/batch_info.rs:196-315): from the
 * running sequences of one step it builds tokens, positions, slot_mapping, logit_idxs, the
 * cu_seqlens of the multi-token entries, gather_mapping, and the block tables and context lengths
 * of the single-token entries.  The reference makes nine Vecs and uploads each with its own
 * Tensor::from_slice(..).to(device); here all sections are written into ONE caller-owned staging
 * buffer (page-locked host memory) at 256-byte aligned offsets and reach the device with ONE
 * cudaMemcpyAsync.  slot_mapping stays int32 (aici_reshape_and_cache accepts it, so the per-layer
 * int64 cast of lib.rs:199-200 is gone). */
typedef struct aici_batch_entry {
  int64_t seq_id;
  const int32_t *tokens;    /* q_len token ids */
  const int64_t *positions; /* q_len positions, or NULL for k_len - q_len .. k_len - 1 */
  const int64_t *kv_slots;  /* k_len cache slots of the whole sequence (block * block_size + off) */
  int32_t q_len;            /* query tokens of this step, >= 1 */
  int32_t k_len;            /* context length including the query tokens, >= q_len */
} aici_batch_entry;

enum {
  AICI_BATCH_PAGED_DECODE = 1,   /* paged_attn_kernel_v > 0: single-token entries go to the back
                                    and get block tables instead of gather_mapping entries */
  AICI_BATCH_TABLES_FOR_ALL = 2, /* block tables and context lengths for the multi-token entries
                                    too (rows 0 .. num_multitoken), for aici_mha_varlen_paged_fwd */
  AICI_BATCH_NO_GATHER_MAP = 4   /* leave gather_mapping empty (nothing calls gather_cached_kv) */
};

typedef struct aici_batch_layout {
  int64_t total_bytes; /* size of the staging buffer and of the device copy */
  /* byte offsets of the sections; element types in the comments */
  int64_t tokens_off;         /* int32 [num_tokens] */
  int64_t positions_off;      /* int64 [num_tokens] */
  int64_t slot_mapping_off;   /* int32 [num_tokens] */
  int64_t logit_idxs_off;     /* int32 [num_entries] */
  int64_t seqlens_q_off;      /* int32 [num_multitoken + 1], offsets into tokens */
  int64_t seqlens_k_off;      /* int32 [num_multitoken + 1] */
  int64_t gather_mapping_off; /* int32 [gather_len] */
  int64_t block_tables_off;   /* int32 [table_rows, max_blocks_per_seq], rows zero-padded */
  int64_t context_lens_off;   /* int32 [table_rows] */
  int32_t num_entries, num_tokens;
  int32_t num_multitoken; /* BatchInfo::seqlen_multi */
  int32_t q_multi;        /* BatchInfo::q_multi: tokens before the first single-token entry */
  int32_t max_seqlen_q, max_seqlen_k;
  int32_t gather_len;
  int32_t num_paged;  /* single-token entries served by the paged decode kernel */
  int32_t table_rows; /* num_paged, or num_entries with AICI_BATCH_TABLES_FOR_ALL */
  int32_t paged_row0; /* first row of the single-token entries in block_tables / context_lens */
  int32_t max_blocks_per_seq;
  int32_t paged_max_context_len;
} aici_batch_layout;

/* Sizes and offsets only; touches no buffer.  Errors mirror the reference's asserts: no entry at
 * all, a position >= max_model_len, a block-start slot that is not a multiple of block_size. */
char *aici_batch_info_layout(const aici_batch_entry *entries, int num_entries, int flags,
                             int block_size, int64_t max_model_len, aici_batch_layout *layout);

/* Fills `staging` (host memory, at least layout->total_bytes; page-locked for an asynchronous
 * copy) and, when device_dst is not NULL, enqueues one host-to-device copy of total_bytes on
 * `stream`.  entry_order[i] (optional, num_entries ints) = index in `entries` of the sequence
 * placed at batch index i, i.e. BatchInfo::seq_id_to_idx inverted.  staging must not be rewritten
 * before the stream has passed the copy. */
char *aici_batch_info_build(const aici_batch_entry *entries, int num_entries, int flags,
                            int block_size, int64_t max_model_len, void *staging,
                            size_t staging_bytes, void *device_dst, size_t device_bytes,
                            aici_batch_layout *layout, int32_t *entry_order, aici_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AICI_B200_H_ */
