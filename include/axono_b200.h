/*
 * axono_b200 - C ABI of the B200 (sm_100a) decode hot path for Axono.
 *
 * Every entry point takes raw device pointers, explicit sizes, a dtype code and a CUDA
 * stream (cudaStream_t passed as void*; NULL = the legacy default stream, which is
 * what the reference's ops launch on outside capture, src/core/cuda/graph.cu:58-62).
 * Every entry point returns an int whose values are those of axono::core::Status
 * (include/axono/core/types.h:54-64); no exception crosses this boundary.  dtype codes
 * are the values of axono::core::DataType (include/axono/core/types.h:18-27).
 *
 * No entry point synchronises the stream, and none allocates device memory, so all of
 * them may be recorded into a CUDA graph (the reference's compile()/CUDAGraph contract,
 * axono/python/axono/core/compile.py:69-174).  Scratch memory is passed in by the caller
 * (see axb200_gqa_workspace_bytes).
 */
#ifndef AXONO_B200_H_
#define AXONO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* axono::core::Status, include/axono/core/types.h:54-64 */
enum {
  AXB200_OK = 0,
  AXB200_INVALID_ARGUMENT = 1,
  AXB200_OUT_OF_MEMORY = 2,
  AXB200_UNSUPPORTED_TYPE = 3,
  AXB200_SHAPE_MISMATCH = 4,
  AXB200_INTERNAL_ERROR = 5,
  AXB200_DEVICE_ERROR = 6,
  AXB200_INVALID_PTR = 7,
  AXB200_DEVICE_MISMATCH = 8
};

/* axono::core::DataType, include/axono/core/types.h:18-27 */
enum {
  AXB200_INT8 = 0,
  AXB200_INT16 = 1,
  AXB200_INT32 = 2,
  AXB200_INT64 = 3,
  AXB200_FLOAT16 = 4,
  AXB200_FLOAT32 = 5,
  AXB200_FLOAT64 = 6,
  AXB200_BOOLEAN = 7
};

/* Bits of the device error word returned by axb200_last_error(). */
enum {
  AXB200_ERR_WAIT_TIMEOUT = 1u,   /* a bounded wait inside a kernel (barrier, peer flag) gave up */
  AXB200_ERR_BAD_PAGE = 2u,       /* a block-table entry was outside [0, num_pages) */
  AXB200_ERR_CAPACITY = 4u,       /* an append found its sequence at capacity, or a decode call found
                                     seq_lens[b] above max_seq_len / the pages (the excess is not read) */
  AXB200_ERR_BAD_INDEX = 8u       /* an embedding id was outside [0, vocab) */
};

const char *axb200_version(void);

/* Reads and clears the error word kernels set instead of trapping (bounded waits that ran
 * out, page ids out of range).  Synchronises the device.  No counterpart in the reference,
 * whose kernels never report (src/ops/cuda/gqa.cu:132-135 ignores launch errors). */
unsigned int axb200_last_error(void);

/* Limit, in nanoseconds of wall time, of every bounded wait inside this library's kernels (a wait
 * on a shared-memory barrier, on a peer GPU's generation flag): a waiter that has polled that long
 * gives up, records AXB200_ERR_WAIT_TIMEOUT and the kernel returns - nothing hangs.  Default 2 s.
 * Launches made afterwards carry the new limit (it travels in the kernel parameters, so a captured
 * graph keeps the limit it was captured with).  After a timeout in a call with peers the ranks'
 * generation counters no longer agree: zero local_state and the flag arrays on every rank before the
 * next such call.  No counterpart in the reference, whose kernels have no waits. */
int axb200_set_wait_limit_ns(uint64_t ns);

/* Who merges the chunk partials of the decode calls.  on (default): the CTA that finishes a
 * (sequence, KV head) last merges and writes the result - one kernel per call; the arrival counters
 * are library-owned device memory (64 regions of 4096 counters, one region per workspace pointer in
 * use, always left zero).  off, or when a call has more than 4096 (sequence, KV head) items or no
 * region is free: a separate combine kernel, as the reference's GqaDecodeMergeKernel
 * (src/ops/cuda/gqa.cu:95-129).  Both forms run the same arithmetic and give identical bits.
 * on == 2: as 1, but the merging CTA takes the query heads of its KV head one at a time instead of
 * two at a time (a tuning switch; same bits again). */
int axb200_set_fused_merge(int on);

/* How a decode call that fits one wave of CTAs is cut into chunks.  on: on the device, from
 * the lengths in device memory (the smallest chunk length for which all chunks fit the wave; every CTA
 * streams about the same bytes).  off (default - it measured faster, the planning costs each CTA
 * about 5 us that nothing hides in a single wave): on the host from max_seq_len alone, one length for all sequences
 * (wave slots / (batch x hkv) chunks each) - the rule the reference's launcher follows in spirit
 * (one split count per call, src/ops/cuda/gqa.cu:157-160).  Both are exact; they differ in speed. */
int axb200_set_device_plan(int on);

/* Whether the decode calls launch their attention kernel as a programmatic dependent of the kernel
 * before it in the stream (default on): its CTAs may then be scheduled while that kernel - the append,
 * in a decode step - is finishing, and stop at a grid-dependency wait until it is complete and its
 * writes are visible; what they do before the wait touches no global memory.  The one-launch decode step
 * (axb200_decode_step_paged) in turn lets the kernel after it be scheduled early, so consecutive steps in a
 * stream or a captured graph overlap launch and set-up with the previous step's tail.  Off: plain stream
 * order.  The result is the same either way.  No counterpart in the reference. */
int axb200_set_dependent_launch(int on);

/* Overrides the chunk length of the decode calls: `tiles` 64-token tiles per chunk (doubled until a
 * sequence of max_seq_len has at most 256 chunks); 0 gives the choice back to the library.  A tuning
 * and test knob: the result does not depend on it beyond rounding.  No counterpart in the reference. */
int axb200_set_chunk_tiles(int tiles);

/* The chunk plan of a decode call, evaluated on the host for lengths given in host memory - the same
 * functions the kernels run on the device lengths.  For each sequence its chunk length in tokens and
 * its number of chunks; max_chunks = partial slots per (sequence, head); grid_ctas = CTAs launched.
 * For tests and capacity planning; the decode calls do not need it.  The reference's plan is
 * n_splits = clamp(ceil(skv / 64), 1, 256) (src/ops/cuda/gqa.cu:157-160). */
int axb200_gqa_chunk_plan(const int32_t *lens_host, int batch, int hq, int hkv, int d, int64_t max_seq_len,
                          int32_t *chunk_tokens_out, int32_t *n_chunks_out, int32_t *max_chunks_out,
                          int32_t *grid_ctas_out);

/* Timing of the dominant kernel alone, for the benchmark's roofline figure: while enabled,
 * every decode call records a CUDA-event pair around its split-kernel launch on the launching
 * stream (up to 4096 calls); collect synchronises the device, returns the summed kernel time and
 * the number of launches, and resets the count.  Not for use during stream capture.  No
 * counterpart in the reference (it has no profiling hooks). */
int axb200_profile_enable(int on);
int axb200_profile_collect(double *split_ms_total, int *launches);

/* ---- decode attention ------------------------------------------------------------------
 * Replaces axono::ops::cuda::GqaDecodeAttention (include/axono/ops/cuda/gqa.h:16-20,
 * src/ops/cuda/gqa.cu:139-182) and its two kernels (split :31-92, merge :95-129).
 * out = softmax(q.K^T / sqrt(d)).V per query head, head h reads KV head h / (hq/hkv);
 * every one of the skv cached tokens is visible (no mask).  fp32 accumulation.
 * dtype: AXB200_FLOAT32 or AXB200_FLOAT16 (q, k, v, out share it).
 */

/* Bytes of scratch the decode calls need for `batch` sequences of up to `max_seq_len` tokens. */
size_t axb200_gqa_workspace_bytes(int batch, int hq, int hkv, int d, int64_t max_seq_len, int dtype);

/* Reference layout, one sequence: q (1,hq,d), k/v (skv,hkv,d) token-major contiguous,
 * out (1,hq,d).  Same contract as libaxono.gqa_decode_attention(q,k,v)
 * (axono/python/src/nanobind_module.cpp:1016-1029). */
int axb200_gqa_decode(const void *q, const void *k, const void *v, void *out,
                      int hq, int hkv, int d, int64_t skv, int dtype,
                      void *workspace, size_t workspace_bytes, void *stream);

/* axb200_gqa_decode without a workspace argument, for callers that must not allocate device
 * memory: a plugin loaded into a host whose allocator owns every byte of the GPU (as the
 * reference's budgeted caching pool does), a serving loop where cudaMalloc's implicit device-wide
 * synchronisation would stall the other streams, or a binding that has the C ABI but no allocator
 * handle.  The split-K partials go into a fixed array inside the library image instead
 * (axb200_static_scratch_bytes() = 4 MiB; each GPU that loads the library holds it until the process
 * exits).  The caller still passes q, k, v and out; same layouts and result as axb200_gqa_decode.
 * Limits and rules:
 *  - returns AXB200_OUT_OF_MEMORY when axb200_gqa_workspace_bytes(1, hq, hkv, d, skv, dtype) exceeds
 *    axb200_static_scratch_bytes() (for 16 query heads and head_dim 128 any skv fits);
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress) with
 *    that device current; make that first call before any stream capture;
 *  - it calls no cudaMalloc / cudaFree and no allocating library routine;
 *  - all calls share the one array, which keeps the previous call's contents.  Nothing in it has
 *    to start at zero (only records written by the same call are read back), but two calls that
 *    overlap on the GPU - different streams, or graphs replayed concurrently - race on it: keep
 *    calls of this entry point ordered on one stream per device.
 * No counterpart in the reference, whose op allocates three workspace tensors per call
 * (src/ops/cuda/gqa.cu:166-168). */
size_t axb200_static_scratch_bytes(void);
int axb200_gqa_decode_static(const void *q, const void *k, const void *v, void *out,
                             int hq, int hkv, int d, int64_t skv, int dtype, void *stream);

/* Batched, paged cache (extension; the reference op has no batch dimension).
 * q/out (batch,hq,d).  k_pages/v_pages: (num_pages, hkv, page_tokens, d), page_tokens a
 * multiple of 64.  block_table int32 (batch, max_blocks): page ids of each sequence in
 * token order.  seq_lens int32 (batch), device memory, read by the kernel (so a captured
 * graph follows a growing cache).  max_seq_len: host-side upper bound of seq_lens, sizes
 * the grid and the scratch; a seq_lens[b] beyond what that bound covers sets AXB200_ERR_CAPACITY
 * and only the covered tokens are attended.  Result b equals axb200_gqa_decode on sequence b's
 * first seq_lens[b] tokens. */
int axb200_gqa_decode_paged(const void *q, void *out, const void *k_pages, const void *v_pages,
                            const int32_t *block_table, const int32_t *seq_lens,
                            int batch, int hq, int hkv, int d,
                            int page_tokens, int max_blocks, int num_pages,
                            int64_t max_seq_len, int dtype,
                            void *workspace, size_t workspace_bytes, void *stream);

/* axb200_gqa_decode_paged under a sliding window: sequence b attends only its last `window` tokens,
 * [max(0, len - window), len); window == 0 means all.  Whole tiles and chunks before the window are
 * never read.  This serves the custom caches the reference's KVCache interface invites (the
 * sliding-window subclass of axono/python/tests/nn/test_kv_cache.py:75-114, which keeps the last W
 * tokens and attends over them). */
int axb200_gqa_decode_paged_window(const void *q, void *out, const void *k_pages, const void *v_pages,
                                   const int32_t *block_table, const int32_t *seq_lens,
                                   int batch, int hq, int hkv, int d,
                                   int page_tokens, int max_blocks, int num_pages,
                                   int64_t max_seq_len, int window, int dtype,
                                   void *workspace, size_t workspace_bytes, void *stream);

/* ---- prefill attention ---------------------------------------------------------------------------------
 * Replaces axono::ops::cuda::ScaledDotProductAttention (include/axono/ops/cuda/sequence.h:37-39,
 * src/ops/cuda/sequence.cu:105-163,451-472): q (sq,hq,d), k/v (skv,hkv,d) token-major, out (sq,hq,d);
 * scale 1/sqrt(d); head h reads KV head h/(hq/hkv); with is_causal row t sees keys [0, t] when
 * skv >= t+1 and every key otherwise (src/ops/cpu/sequence.cpp:269-270).  fp16 with d == 128 runs on
 * the tcgen05 tensor cores; FLOAT32 and other head sizes (d a multiple of 4 up to 192, sq >= 16) on a
 * tiled FMA kernel with fp32 arithmetic; neither needs scratch.  The remaining cases run row by row
 * on the decode kernels and need axb200_sdpa_workspace_bytes of scratch (0 for the first two).
 * There is no shared-memory limit on skv. */
size_t axb200_sdpa_workspace_bytes(int sq, int hq, int hkv, int d, int64_t skv, int dtype);
int axb200_sdpa(const void *q, const void *k, const void *v, void *out,
                int sq, int hq, int hkv, int d, int64_t skv, int is_causal, int dtype,
                void *workspace, size_t workspace_bytes, void *stream);

/* ---- decode attention fused with the all-gather of per-head outputs ------------------------------
 * For KV heads sharded over `world` GPUs of one node (one process per GPU): rank `rank` holds hkv KV
 * heads and the hq matching query heads of every sequence.  Same computation as
 * axb200_gqa_decode_paged on the local heads, but the combine kernel stores each merged row straight
 * into EVERY rank's gathered buffer (batch, hq_total, d) at head rank*hq + h - plain stores through
 * peer-mapped pointers over NVLink - then exchanges generation flags with the peers (bounded wait,
 * AXB200_ERR_WAIT_TIMEOUT on expiry), so that when the call's last kernel completes the local
 * gathered buffer holds all heads.  It replaces "attention, then ncclAllGather" by one kernel pair.
 *   peer_out[r], peer_flags[r]: host arrays of `world` device pointers - rank r's gathered buffer for
 *     this call and rank r's flag array (world x uint32), mapped into this process (own entries are
 *     local pointers); local_state: 2 x uint32 of this rank.  All zero-initialised once.
 *   Successive calls must alternate between at least two gathered buffers (e.g. one per layer), and
 *   every rank must make the same sequence of calls.  No counterpart in the reference (single GPU). */
int axb200_gqa_decode_paged_gather(const void *q, const void *k_pages, const void *v_pages,
                                   const int32_t *block_table, const int32_t *seq_lens,
                                   int batch, int hq, int hkv, int d,
                                   int page_tokens, int max_blocks, int num_pages,
                                   int64_t max_seq_len, int dtype,
                                   void *workspace, size_t workspace_bytes,
                                   void *const *peer_out, void *const *peer_flags, void *local_state,
                                   int world, int rank, int hq_total, void *stream);

/* Context-parallel decode: the tokens of every sequence are spread over `world` GPUs (any split -
 * softmax does not depend on token order; keys are rotated with their global positions before they are
 * cached).  Each rank attends its share; its combine kernel stores an un-normalised record
 * [O(d), m, l] per (sequence, head) into every rank's record buffer (batch, hq, world, d + 2) fp32
 * and exchanges generation flags as above; a merge kernel then forms the same `out` (batch,hq,d) on
 * every rank from local memory.  For one very long sequence that neither batch nor head sharding
 * can spread.  peer_records / peer_flags / local_state as in axb200_gqa_decode_paged_gather; successive
 * calls must alternate between at least two record buffers.  No counterpart in the reference. */
int axb200_gqa_decode_paged_cp(const void *q, void *out, const void *k_pages, const void *v_pages,
                               const int32_t *block_table, const int32_t *seq_lens,
                               int batch, int hq, int hkv, int d,
                               int page_tokens, int max_blocks, int num_pages,
                               int64_t max_seq_len, int dtype,
                               void *workspace, size_t workspace_bytes,
                               void *const *peer_records, void *const *peer_flags, void *local_state,
                               int world, int rank, void *stream);

/* ---- the same gather as a library collective (NCCL) ---------------------------------------------------
 * "Attention, then all-gather of the per-head outputs, then the output projection" with ncclAllGather:
 * the plain form of KV-head sharding and the baseline of the fused kernel above.  One process per GPU.
 *   unique_id: rank 0 draws 128 bytes and sends them to the other ranks by any host-side means;
 *   init: creates this rank's communicator and runs one small collective on it - it allocates and
 *     synchronises, so every rank calls it before any stream capture;
 *   all_gather: every rank contributes bytes_per_rank bytes at `send` and receives world x that at
 *     `recv`, rank-major; only enqueues on `stream`, so it may be captured into a CUDA graph (every
 *     rank must then replay its graph the same number of times);
 *   swap_leading_dims: dst (n1, n0, row) = src (n0, n1, row), rows of row_bytes (a multiple of 16,
 *     pointers 16-byte aligned) - turns the gathered (world, batch, heads x d) into the
 *     (batch, world, heads x d) rows the projection reads.
 * Destroy a communicator only after every CUDA graph that recorded one of its all-gathers has been
 * destroyed: ncclCommDestroy waits for them (a live graph makes the call block for good).
 * NCCL is opened by soname (libnccl.so.2) on first use.  No counterpart in the reference, whose
 * WITH_NCCL option is reserved and unused (CMakeLists.txt:78,91-92). */
int axb200_nccl_unique_id(void *id128);
int axb200_nccl_init(const void *id128, int world, int rank, void **comm_out);
int axb200_nccl_all_gather(void *comm, const void *send, void *recv, size_t bytes_per_rank, void *stream);
int axb200_nccl_destroy(void *comm);
int axb200_swap_leading_dims(const void *src, void *dst, int n0, int n1, size_t row_bytes, void *stream);

/* Peer-mappable device memory for the calls above (CUDA IPC): alloc returns zero-filled memory and a
 * 64-byte handle to send to the other processes of the node; open maps a peer's handle; close
 * unmaps it; free releases an allocation.  These four are set-up calls: they allocate and
 * synchronise, unlike every other entry point.  No counterpart in the reference. */
int axb200_p2p_alloc(size_t bytes, void **dev_ptr, void *handle64);
int axb200_p2p_open(const void *handle64, void **dev_ptr);
int axb200_p2p_close(void *dev_ptr);
int axb200_p2p_free(void *dev_ptr);

/* ---- KV-cache append with RoPE / M-RoPE --------------------------------------------------
 * Replaces, for one decode step of `batch` sequences, the reference's per-layer sequence
 *   rope|rope_thd(q), rope|rope_thd(k)      (src/ops/cuda/sequence.cu:318-342, 421-449)
 *   cache.update -> concat(old, new, axis 0) (axono/python/axono/nn/kv_cache.py:96-102,
 *                                             src/ops/cuda/sequence.cu:474-521)
 * by one launch: q (batch,hq,d) is rotated in place, k_new (batch,hkv,d) is rotated and
 * written, v_new copied, into slot seq_lens[b] + slot_delta of sequence b's pages; when `advance`
 * is non-zero seq_lens[b] is then incremented.  All layers of a model share seq_lens: the first
 * layer of a step appends with slot_delta 0 and advance 1 (so every layer's attention sees the new
 * token), the other layers with slot_delta -1 and advance 0.  Rotation: rotate-half pairs (i, i+d/2).
 *   mrope == 0: angle_i = float(pos[b]) * inv_freq[i];   pos int64 (batch)
 *   mrope != 0: pos int64 (3,batch) rows T,H,W; pair i uses H when i%3==1 && i<3*h_sec,
 *               W when i%3==2 && i<3*w_sec, else T (src/ops/cpu/sequence.cpp:222-227).
 * pos == NULL: the position is the slot index (the cache length before the append) on every axis.
 * inv_freq: device float (d/2), or NULL to use theta^(-2i/d) computed on the host with the
 * C library's powf, exactly as the reference's CPU Rope does (src/ops/cpu/sequence.cpp:83-84).
 * rotate == 0 skips the rotation (plain append).
 */
int axb200_kv_append_rope(void *q, const void *k_new, const void *v_new,
                          void *k_pages, void *v_pages,
                          const int32_t *block_table, int32_t *seq_lens,
                          const int64_t *pos, const float *inv_freq, float theta,
                          int rotate, int mrope, int h_sec, int w_sec,
                          int batch, int hq, int hkv, int d,
                          int page_tokens, int max_blocks, int num_pages,
                          int dtype, int slot_delta, int advance, void *stream);

/* Prefill side of the cache: writes n tokens of ONE sequence - k, v (n,hkv,d) token-major - into its
 * pages at slots start .. start+n-1 (block_row = the sequence's row of the block table), rotating k
 * (and q (n,hq,d) in place, when given) with each token's own position: pos int64 (n), or (3,n) with
 * mrope, or NULL for start + i.  It replaces rope|rope_thd over the prompt followed by the first
 * cache.update (axono/python/examples/vlm/qwen3vl/model.py:358-362,
 * axono/python/axono/nn/kv_cache.py:96-100).  The caller sets the sequence's length afterwards. */
int axb200_kv_prefill_write(void *q, const void *k, const void *v, void *k_pages, void *v_pages,
                            const int32_t *block_row, const int64_t *pos, const float *inv_freq,
                            float theta, int rotate, int mrope, int h_sec, int w_sec,
                            int64_t n, int hq, int hkv, int d,
                            int page_tokens, int max_blocks, int num_pages, int64_t start,
                            int dtype, void *stream);

/* The same step taken straight from the QKV projection's output, with the per-head RMS norms the
 * reference's text tower applies in between (axono/python/examples/vlm/qwen3vl/model.py:353-362:
 * reshape, rms_norm(q, q_norm), rms_norm(k, k_norm), rope_thd / rope on q and k, cache.update): one
 * launch replaces those six.  qkv (batch, ld): each row holds hq query heads, then hkv key heads, then
 * hkv value heads of d elements; q_norm_w / k_norm_w (d) or NULL (no norm); the normed, rotated q
 * goes to q_out (batch,hq,d), k and v into the page slot.  Other arguments as above. */
int axb200_qkv_norm_rope_append(const void *qkv, int64_t ld, const void *q_norm_w, const void *k_norm_w,
                                float eps, void *q_out, void *k_pages, void *v_pages,
                                const int32_t *block_table, int32_t *seq_lens,
                                const int64_t *pos, const float *inv_freq, float theta,
                                int rotate, int mrope, int h_sec, int w_sec,
                                int batch, int hq, int hkv, int d,
                                int page_tokens, int max_blocks, int num_pages,
                                int dtype, int slot_delta, int advance, void *stream);

/* One decode step of one layer as one operator: what the reference's layer does with three calls per
 * token - rope on q and k, cache.update, gqa_decode_attention
 * (axono/python/examples/vlm/qwen3vl/model.py:358-366) - i.e. axb200_kv_append_rope (slot_delta 0,
 * advance 1) followed by axb200_gqa_decode_paged, with the same arguments and the same results bit for
 * bit, except that q is only read: the rotated q never leaves the kernel (or, in the two-launch form,
 * goes to the workspace).  For fp16 with head_dim 64 or 128 this is ONE launch: the attention kernel reads
 * the old length, works with length + 1, rotates q in registers, and the CTA that owns the new token's
 * row rotates k_new, stores k and v to the page and puts them into its staged tile; the last CTA of a
 * sequence to have read the old length stores the new one.  Other types and head sizes run the two
 * kernels.  max_seq_len bounds the lengths AFTER the append.  A sequence without room for the token sets
 * AXB200_ERR_CAPACITY, appends nothing and attends its old tokens.  workspace: at least
 * axb200_decode_step_workspace_bytes, 16-byte aligned; calls that may overlap on the GPU use different
 * workspaces.  axb200_decode_step_launches: 1 or 2, how many kernels the call launches for these sizes
 * (aligned pointers assumed).  axb200_set_step_fused(0) forces the two-launch form (A/B, tests). */
size_t axb200_decode_step_workspace_bytes(int batch, int hq, int hkv, int d, int64_t max_seq_len, int dtype);
int axb200_decode_step_launches(int batch, int hq, int hkv, int d, int64_t max_seq_len, int dtype);
int axb200_set_step_fused(int on);
int axb200_decode_step_paged(const void *q, const void *k_new, const void *v_new, void *out,
                             void *k_pages, void *v_pages, const int32_t *block_table, int32_t *seq_lens,
                             const int64_t *pos, const float *inv_freq, float theta,
                             int rotate, int mrope, int h_sec, int w_sec,
                             int batch, int hq, int hkv, int d,
                             int page_tokens, int max_blocks, int num_pages, int64_t max_seq_len,
                             int dtype, void *workspace, size_t workspace_bytes, void *stream);

/* The same one-operator step taken straight from the QKV projection's output, for the text tower's layer
 * (axono/python/examples/vlm/qwen3vl/model.py:353-366: reshape, rms_norm(q), rms_norm(k), rope on both,
 * cache.update, gqa_decode_attention): axb200_qkv_norm_rope_append followed by the paged decode attention,
 * same arguments, same results bit for bit - one launch for fp16 with head_dim 64 / 128, the two kernels
 * otherwise (the normed, rotated q then goes to the workspace).  slot_delta / advance: (0, 1) for the first
 * layer of a step, (-1, 0) for the later ones, as in axb200_kv_append_rope.  world == 0: the result goes to
 * out (batch,hq,d).  world > 0: heads are sharded over `world` ranks and the rows go into every rank's
 * gathered buffer with the flag exchange of axb200_gqa_decode_paged_gather (same peer arguments; out unused).
 * workspace: at least axb200_decode_step_workspace_bytes. */
int axb200_qkv_decode_step_paged(const void *qkv, int64_t ld, const void *q_norm_w, const void *k_norm_w, float eps,
                                 void *out, void *k_pages, void *v_pages, const int32_t *block_table,
                                 int32_t *seq_lens, const int64_t *pos, const float *inv_freq, float theta,
                                 int rotate, int mrope, int h_sec, int w_sec, int batch, int hq, int hkv, int d,
                                 int page_tokens, int max_blocks, int num_pages, int64_t max_seq_len, int dtype,
                                 int slot_delta, int advance, void *workspace, size_t workspace_bytes,
                                 void *const *peer_out, void *const *peer_flags, void *local_state, int world,
                                 int rank, int hq_total, void *stream);

/* One decode step with HOST activations: copies q (batch,hq,d), k_new, v_new (batch,hkv,d) from host
 * (pinned memory for asynchronous copies) into the device staging buffers q_dev / k_new_dev /
 * v_new_dev, runs axb200_kv_append_rope (slot_delta 0, advance 1) and axb200_gqa_decode_paged, copies
 * the attention output (batch,hq,d) to out_host and waits for it on `stream`.  This is the step the
 * reference's host loop performs through its binding each token
 * (axono/python/examples/vlm/qwen3vl/model.py:738-761), as a single call.  The cache, block table,
 * lengths, positions and scratch stay device-resident as in the two calls it composes. */
int axb200_decode_step_host(const void *q_host, const void *k_new_host, const void *v_new_host,
                            void *out_host, void *q_dev, void *k_new_dev, void *v_new_dev, void *out_dev,
                            void *k_pages, void *v_pages, const int32_t *block_table, int32_t *seq_lens,
                            const int64_t *pos, const float *inv_freq, float theta,
                            int rotate, int mrope, int h_sec, int w_sec,
                            int batch, int hq, int hkv, int d,
                            int page_tokens, int max_blocks, int num_pages,
                            int64_t max_seq_len, int dtype,
                            void *workspace, size_t workspace_bytes, void *stream);

/* ---- RoPE family (stand-alone ops) --------------------------------------------------------
 * x/out (rows,heads,dim); out may alias x. */

/* axono::ops::cuda::Rope, include/axono/ops/cuda/sequence.h, src/ops/cuda/sequence.cu:318-342;
 * pos int64 (rows). */
int axb200_rope(const void *x, const int64_t *pos, float theta, void *out,
                int64_t rows, int heads, int dim, int dtype, void *stream);

/* axono::ops::cuda::RopeThd, src/ops/cuda/sequence.cu:421-449; pos int64 (3,rows),
 * inv_freq float (dim/2); t_sec is accepted and ignored as in the reference (:425). */
int axb200_rope_thd(const void *x, const int64_t *pos, const float *inv_freq,
                    int t_sec, int h_sec, int w_sec, void *out,
                    int64_t rows, int heads, int dim, int dtype, void *stream);

/* axono::ops::cuda::RopeWithCosSin, src/ops/cuda/sequence.cu:344-367; cos/sin float (rows,dim). */
int axb200_rope_with_cos_sin(const void *x, const float *cos_t, const float *sin_t, void *out,
                             int64_t rows, int heads, int dim, int dtype, void *stream);

/* axono::ops::cuda::MropeCosSin, src/ops/cuda/sequence.cu:372-419; pos int64 (3,rows),
 * inv_freq float (half); cos/sin out float (rows, 2*half). */
int axb200_mrope_cos_sin(const int64_t *pos, const float *inv_freq, int h_sec, int w_sec,
                         float *cos_out, float *sin_out, int64_t rows, int half, void *stream);

/* ---- fused norm / activation ---------------------------------------------------------------*/

/* axono::ops::cuda::AddRmsNorm, include/axono/ops/cuda/fused.h:14-25, src/ops/cuda/fused.cu:91-110:
 * y = x + residual; out = y * rsqrt(mean(y^2) + eps) * weight.  x/residual/y/out (rows,hidden),
 * weight (hidden), all of `dtype`; fp32 math. */
int axb200_add_rms_norm(const void *x, const void *residual, const void *weight, float eps,
                        void *y, void *out, int64_t rows, int hidden, int dtype, void *stream);

/* axono::ops::cuda::SiluMul, src/ops/cuda/fused.cu:76-89: out = gate / (1 + exp(-gate)) * up. */
int axb200_silu_mul(const void *gate, const void *up, void *out, int64_t n, int dtype, void *stream);

/* SiluMul on the two halves of one matrix - the output of a fused gate|up projection
 * (model.py:383-384 calls silu_mul(gate_proj(x), up_proj(x))): gate = in[r, 0:n], up = in[r, n:2n],
 * row stride ld; out (rows, n).  Saves the two slicing copies. */
int axb200_silu_mul_rows(const void *gate_up, int64_t ld, int n, int64_t rows, void *out, int dtype,
                         void *stream);

/* axono::ops::cuda::RmsNorm, include/axono/ops/cuda/llm.h:33-36, src/ops/cuda/llm.cu:345-373:
 * out = x * rsqrt(mean(x^2) + eps) * weight over the last dim; weight may be NULL. */
int axb200_rms_norm(const void *x, const void *weight, float eps, void *out,
                    int64_t rows, int cols, int dtype, void *stream);

/* axono::ops::cuda::Embedding, src/ops/cuda/sequence.cu:75-81,294-316: out[i] = table[ids[i]];
 * ids int32 or int64 (n), table (vocab, hidden) of `dtype`, out (n, hidden).  An id outside the table
 * sets AXB200_ERR_BAD_INDEX and gives a zero row (the reference reads out of bounds). */
int axb200_embedding(const void *ids, int ids_dtype, const void *table, void *out, int64_t n,
                     int64_t vocab, int hidden, int dtype, void *stream);

/* axono::ops::cuda::ArgmaxLastDim, src/ops/cuda/sequence.cu:262-292,560-581, with the tie rule of the
 * reference's CPU op (src/ops/cpu/sequence.cpp:370-400): the lowest index among equal maxima.
 * x (rows, cols) of `dtype`, out int64 (rows). */
int axb200_argmax_last_dim(const void *x, int64_t *out, int64_t rows, int cols, int dtype, void *stream);

/* Half2FloatKernel / Float2HalfKernel (src/core/cuda/tensor/kernel.cu:175-193), the device side of
 * Tensor::CastTo: FLOAT16 <-> FLOAT32, IEEE round to nearest even. */
int axb200_cast(const void *src, int src_dtype, void *dst, int dst_dtype, int64_t n, void *stream);

/* out[i] = mean + stddev * N(0,1), i < n, from a counter-based generator: the values depend only on
 * (seed, i).  Stands where the reference has its randn operator (src/ops/cuda/randn.cu:13-32, cuRAND
 * seeded from std::random_device - not repeatable); used to fill KV pages for benchmarks and tests. */
int axb200_randn(void *out, int64_t n, int dtype, float mean, float stddev, uint64_t seed, void *stream);

/* The tower's projection: out (rows, out_features) = x (rows, in_features) . w (out_features,
 * in_features)^T as ONE cuBLASLt call (FLOAT16 with fp32 accumulation, or FLOAT32) - a library GEMM, as
 * the reference's LinearNoBias is (src/ops/cuda/linear.cu:105-203); outside the rewritten path.  The
 * first call of a shape (outside any stream capture) times up to eight heuristic candidates on the
 * operands given and keeps the fastest; later calls, captured or not, reuse it.  All calls on a device
 * share one library workspace: keep them ordered on one stream per device. */
int axb200_linear_nobias(const void *x, const void *w, void *out, int64_t rows, int64_t out_features,
                         int64_t in_features, int dtype, void *stream);

/* axono::ops::cuda::Concat, src/ops/cuda/sequence.cu:474-521, on bytes: out (outer, a_bytes +
 * b_bytes) = a (outer, a_bytes) ++ b (outer, b_bytes).  Axis 0 is outer == 1. */
int axb200_concat(const void *a, const void *b, void *out, int64_t outer,
                  size_t a_bytes, size_t b_bytes, void *stream);

/* ---- KV page arena ---------------------------------------------------------------------------------
 * The allocator side of the paged cache: fixed per-layer K/V pools of pages with a free list, one
 * block table (max_seqs, max_blocks) and one length vector (max_seqs) shared by all layers.  It
 * replaces the reference's handling of KV tensors - a fresh, ever larger allocation from the
 * size-bucketed caching pool on every concat (axono/python/axono/nn/kv_cache.py:96-102,
 * src/core/cuda/detail.cu:41-146,153-275).  Pools are allocated and zero-filled once, keep their
 * addresses (graph replay), are never evicted and never re-zeroed on reuse.  A sequence slot is the
 * batch row the decode kernels see: pass batch = max_seqs; rows not in use have length 0.
 * Host-side and thread-safe; with device_memory == 0 only the bookkeeping exists (no CUDA calls).
 * These are set-up / between-step calls: create and destroy allocate and synchronise. */
typedef struct axb200_kv_arena axb200_kv_arena;
int axb200_kv_arena_create(int n_layers, int num_pages, int hkv, int page_tokens, int d, int dtype,
                           int max_seqs, int max_blocks, int device_memory, axb200_kv_arena **out);
int axb200_kv_arena_destroy(axb200_kv_arena *arena);
/* Takes the lowest free sequence slot and pages for reserve_tokens; OUT_OF_MEMORY when slots or
 * pages run out (nothing is taken then). */
int axb200_kv_arena_alloc_seq(axb200_kv_arena *arena, int64_t reserve_tokens, int *seq_id);
/* Grows the sequence to hold `tokens` tokens in total (all or nothing). */
int axb200_kv_arena_reserve(axb200_kv_arena *arena, int seq_id, int64_t tokens);
/* Permutes the free list with a seeded generator, so that the pages handed out next are scattered over
 * the pools the way they are in an arena that has served many sequences.  Benchmarks and tests use it
 * to run on non-contiguous page tables. */
int axb200_kv_arena_shuffle_free(axb200_kv_arena *arena, uint64_t seed);
/* Returns the pages to the free list and zeroes the device-side length on `stream`. */
int axb200_kv_arena_free_seq(axb200_kv_arena *arena, int seq_id, void *stream);
/* Uploads the block-table rows changed since the last sync (one H2D copy on `stream`). */
int axb200_kv_arena_sync(axb200_kv_arena *arena, void *stream);
int axb200_kv_arena_stats(axb200_kv_arena *arena, int64_t *pages_total, int64_t *pages_free,
                          int64_t *seqs_live, int64_t *device_bytes);
/* Copies the sequence's page ids (host view) into pages_out; returns how many it holds, -1 on error. */
int axb200_kv_arena_seq_pages(axb200_kv_arena *arena, int seq_id, int32_t *pages_out, int capacity);
int axb200_kv_arena_geometry(axb200_kv_arena *arena, int *n_layers, int *num_pages, int *hkv, int *page_tokens,
                             int *d, int *dtype, int *max_seqs, int *max_blocks);
void *axb200_kv_arena_k_pages(axb200_kv_arena *arena, int layer);
void *axb200_kv_arena_v_pages(axb200_kv_arena *arena, int layer);
int32_t *axb200_kv_arena_block_table(axb200_kv_arena *arena);
int32_t *axb200_kv_arena_seq_lens(axb200_kv_arena *arena);

#ifdef __cplusplus
}
#endif
#endif /* AXONO_B200_H_ */
