/*
 * streamattn_b200 - C ABI of the B200 (sm_100a) decode-attention library.
 *
 * This is the drop-in boundary: plain pointers, sizes and a CUDA stream handle,
 * no torch types.  Every entry point names the reference interface it replaces
 * (paths inside the StreamAttn project).  All device pointers must belong to
 * the device that is current on the calling thread; kernels are enqueued on
 * `stream` and the calls return without synchronising.  Return value: SA_OK or
 * an SA_ERR_* code; sa_last_error() then holds a message (thread-local).
 *
 * Tensors (D = head_dim contiguous in every tensor):
 *   q        [batch, q_heads, D]        addressed by q_stride_b / q_stride_h (elements)
 *   out      [batch, q_heads, D]        contiguous, same dtype as q      (SA_OUT_FINAL)
 *            [batch, q_heads, D+2] f32  (o unnormalised, m, l)           (SA_OUT_STATE)
 *            m is the running maximum of score*scale*log2(e) (base-2 domain),
 *            l = sum 2^(s-m), o = sum 2^(s-m) v.
 *   GQA map  kv_head = q_head / (q_heads / kv_heads)
 *   scale    1/sqrt(D)
 */
#ifndef STREAMATTN_B200_H_
#define STREAMATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SA_API __attribute__((visibility("default")))
#else
#define SA_API
#endif

typedef void *sa_stream_t; /* cudaStream_t */
typedef struct sa_plan sa_plan_t; /* bound plan, see the end of this header */

enum sa_status {
    SA_OK = 0,
    SA_ERR_INVALID = 1,     /* bad argument (maps to ValueError)                    */
    SA_ERR_UNSUPPORTED = 2, /* valid but outside what the kernels cover             */
    SA_ERR_CUDA = 3,        /* CUDA runtime / driver error (maps to RuntimeError)   */
    SA_ERR_DEVICE = 4       /* no sm_100 device / driver entry point missing        */
};

enum sa_dtype { SA_DTYPE_BF16 = 0, SA_DTYPE_F16 = 1, SA_DTYPE_F32 = 2 };
enum sa_index_dtype { SA_INDEX_I32 = 0, SA_INDEX_I64 = 1 };
enum sa_page_layout { SA_LAYOUT_NHD = 0, SA_LAYOUT_HND = 1 };
enum sa_block_order { SA_ORDER_SEQUENTIAL = 0, SA_ORDER_RECENT_FIRST = 1, SA_ORDER_SINK_RECENT_FIRST = 2 };
enum sa_out_mode { SA_OUT_FINAL = 0, SA_OUT_STATE = 1 };
enum sa_kernel_choice { SA_KERNEL_AUTO = 0, SA_KERNEL_STREAM = 1, SA_KERNEL_GENERIC = 2 };
/* May be OR-ed into any kernel_choice argument.  The streaming kernel then lets the CTAs that
   share a (row, KV head) pair claim their tiles from a device counter instead of owning a fixed
   slice, which evens out SMs that the memory system serves at different rates (a few percent
   faster on HBM-bound calls).  The split states are then grouped differently from launch to
   launch, so results agree within the float tolerance but are not bit-reproducible; without
   the flag every call with the same inputs returns the same bits.  Ignored where it does not
   apply (generic kernel, fewer than four CTAs per pair, very long rows). */
#define SA_KERNEL_FLAG_DYNAMIC 0x100

/* Bits of the device status word (sa_workspace_status). */
enum sa_device_status {
    SA_DEV_OK = 0,
    SA_DEV_PIPELINE_TIMEOUT = 1, /* a bounded wait (copy barrier, split states in
                                    flight, a peer rank's state) gave up: the output
                                    is incomplete and the workspace must be
                                    zero-filled again before its next use          */
    SA_DEV_BAD_PAGE = 2          /* an active page_table entry was out of range and
                                    was skipped (never dereferenced)                */
};

#define SA_MAX_SEED_BLOCKS 256

/* Library / device queries. No reference counterpart beyond the capability
 * gate torch.cuda.get_device_capability() == (9, 0) in
 * stream_attention/backends/sm90/transposed_gqa_exact.py:254 and paged.py:320;
 * here the gate is compute capability 10.x. */
SA_API int sa_version(void);
SA_API const char *sa_last_error(void);
SA_API int sa_device_supported(int device);
SA_API int sa_device_sm_count(int device);

/* Workspace (fp32 split states + arrival counters + status word) every decode
 * call needs.  Replaces the partial_o / partial_lse allocation of
 * ExactDecodePlan.build (backends/sm90/transposed_gqa_exact.py:332-347) and
 * make_paged_exact_workspace (kernels/paged_exact_triton.py:309-331).
 * The buffer must be zero-filled ONCE before its first use; calls leave it
 * ready (all zero behind the status word) for the next call, unless a call
 * reported SA_DEV_PIPELINE_TIMEOUT: then zero-fill it again.  Concurrent calls
 * must not share a workspace.
 * num_ctas: 0 = automatic.  Depends only on its arguments (no device query). */
SA_API size_t sa_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim, int num_ctas);

/* Synchronise `stream` and return the sa_device_status bits recorded by the
 * kernels that used `workspace` (then clear them).  Negative on CUDA errors. */
SA_API int sa_workspace_status(void *workspace, sa_stream_t stream);

/*
 * Exact contiguous GQA decode: out = softmax(q K^T / sqrt(D)) V over tokens
 * [0, len_b) of each row, one query token per row, split-KV with an exact
 * (m, l, o) merge fused into the same launch.
 * Replaces exact_decode_out / exact_partial_out + exact_merge_warp_out
 * (backends/sm90/transposed_gqa_exact_sources.py:100-132, 1003-1522) and
 * exact_decode_attention_rows_triton_forward_out_bhnd
 * (kernels/gate0_exact_refresh_triton.py:266-344).
 * k/v: token n of kv head h of row b at  b*kv_stride_b + n*kv_stride_n + h*kv_stride_h
 * (elements), which covers BNHD [B,N,Hkv,D] and head-major [B,Hkv,N,D].
 * seq_lens: optional device array [batch] (lens_dtype) of valid token counts,
 * clipped to kv_len (the reference's cache_position+1); NULL = kv_len.
 */
SA_API int sa_exact_decode(const void *q, const void *k, const void *v, void *out,
                           void *workspace, size_t workspace_bytes,
                           const void *seq_lens, int lens_dtype,
                           int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                           int64_t q_stride_b, int64_t q_stride_h,
                           int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                           int dtype, int out_mode, int num_ctas, int kernel_choice,
                           sa_stream_t stream);

/*
 * sa_exact_decode_static - sa_exact_decode for callers that must not allocate.
 * It has no counterpart in the reference.
 *
 * Some callers cannot obtain a workspace: code running under an allocator that
 * was handed all of the GPU's memory at start-up (a serving engine that gives
 * every free byte to its KV-cache pool, so a later cudaMalloc fails), code on a
 * path where an allocation would synchronise the device (inside a latency-bound
 * decode loop), or a plugin that is only ever given the tensors of the call.
 * For them the split states, arrival counters and status word live in a fixed
 * array inside the library's device image (SA_STATIC_SCRATCH_BYTES, 2 MiB, held
 * by every GPU that loads the library for the life of the process).  The call
 * takes the same arguments as sa_exact_decode minus the workspace and computes
 * the same result with the same kernels.  It calls no cudaMalloc, cudaFree or
 * other allocating routine.
 *
 * Limits and rules:
 *  - shapes whose split states do not fit the array are refused with
 *    SA_ERR_UNSUPPORTED (nothing is launched); use sa_exact_decode then.
 *    With num_ctas = 0 the need is about
 *    512 + 4*batch*q_heads + 4*(148 + batch*kv_heads)*(q_heads/kv_heads)*(head_dim+4) bytes;
 *  - the first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress, with that device current); make that first call
 *    outside any stream capture;
 *  - all calls on a device share the one array: calls that may overlap on the
 *    GPU (different streams) race and give wrong results.  Calls on one stream
 *    are safe; each call clears the arrival counters it needs before launching
 *    (one small cudaMemsetAsync on `stream` that the workspace entry points do
 *    not pay);
 *  - the device status bits of these calls collect in the array's status word;
 *    read them with sa_static_status(), as sa_workspace_status() does for a
 *    caller-provided workspace.
 */
#define SA_STATIC_SCRATCH_BYTES (2 * 1024 * 1024)
SA_API int sa_exact_decode_static(const void *q, const void *k, const void *v, void *out,
                                  const void *seq_lens, int lens_dtype,
                                  int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                                  int64_t q_stride_b, int64_t q_stride_h,
                                  int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                  int dtype, int out_mode, int num_ctas, int kernel_choice,
                                  sa_stream_t stream);
/* Status of the sa_exact_decode_static calls on the current device (no counterpart in the
 * reference; allocates nothing): synchronise `stream`, return the sa_device_status bits collected
 * since the last query and clear them.  A non-zero result also re-zeroes the built-in array, so
 * the next call starts clean.  Negative on CUDA errors.  Without this query a wait that gave up
 * would go unnoticed: the decode call itself returns before the kernel has run. */
SA_API int sa_static_status(sa_stream_t stream);

/*
 * Paged exact decode over a page pool with a page table and ragged per-row
 * lengths.  Replaces paged_exact_decode_out, paged_fragmented_exact_decode_out,
 * paged_fragmented_ragged_exact_decode_out
 * (backends/sm90/transposed_gqa_exact_sources.py:116-132, 2082-2360) and
 * paged_exact_decode_triton_forward_out (kernels/paged_exact_triton.py:193-306).
 * k_pages/v_pages: NHD [num_pages, page_size, kv_heads, D] or
 * HND [num_pages, kv_heads, page_size, D], contiguous.
 * page_table [batch, max_pages_per_request] (table_dtype), -1 marks inactive
 * trailing slots which are never read; seq_lens [batch] (lens_dtype).
 * trace: optional device int32 [batch, max_pages_per_request]; when non-NULL
 * the kernel records the physical page it loaded for every logical page it
 * visited (other slots untouched) - the page-table walk, for parity checks.
 */
SA_API int sa_paged_decode(const void *q, const void *k_pages, const void *v_pages,
                           const void *page_table, const void *seq_lens, void *out,
                           void *workspace, size_t workspace_bytes, int32_t *trace,
                           int batch, int q_heads, int kv_heads, int head_dim,
                           int page_size, int max_pages_per_request, int64_t num_pages,
                           int layout, int dtype, int table_dtype, int lens_dtype,
                           int out_mode, int num_ctas, int kernel_choice, sa_stream_t stream);

/*
 * Seed block rule (host integer logic, no GPU needed).  Writes the seed blocks
 * in the reference's order (sink, recent, middle; duplicates and out-of-range
 * blocks dropped) and returns their count, or -1 if capacity is too small.
 * Replaces policy_seed_blocks (seed_selectors.py:77-104), which equals the
 * in-kernel rule of kernels/gate0_seed_only_triton.py:64-79.
 */
SA_API int sa_seed_blocks(int64_t kv_len, int block_size, int sink_blocks, int recent_blocks,
                          int middle_seed_blocks, int block_order, int32_t *blocks_out, int capacity);

/* Token set of a block list: block*bs + [0,bs) clipped to kv_len, deduplicated,
 * ascending.  Returns the count or -1.  Replaces seed_token_indices_from_blocks
 * (seed_selectors.py:152-173) / seed_indices (:107-133). */
SA_API int64_t sa_seed_token_indices(int64_t kv_len, int block_size, const int32_t *blocks,
                                     int num_blocks, int64_t *tokens_out, int64_t capacity);

/*
 * Seed-only decode: exact attention restricted to the seed token set, K/V shared
 * by the query heads of a KV group (each seed token is read once per KV head).
 * Replaces gate0_seed_only_attention_triton_forward_out[_prechecked]
 * (kernels/gate0_seed_only_triton.py:30-127, 1458-1537, 2322-2378).
 * sa_seed_decode derives the blocks from the policy parameters with
 * sa_seed_blocks; sa_seed_decode_blocks takes an explicit HOST block list
 * (<= SA_MAX_SEED_BLOCKS entries, any order, duplicates ignored).
 */
SA_API int sa_seed_decode(const void *q, const void *k, const void *v, void *out,
                          void *workspace, size_t workspace_bytes,
                          int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                          int64_t q_stride_b, int64_t q_stride_h,
                          int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                          int dtype, int block_size, int sink_blocks, int recent_blocks,
                          int middle_seed_blocks, int block_order,
                          int num_ctas, int kernel_choice, sa_stream_t stream);

SA_API int sa_seed_decode_blocks(const void *q, const void *k, const void *v, void *out,
                                 void *workspace, size_t workspace_bytes,
                                 int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                                 int64_t q_stride_b, int64_t q_stride_h,
                                 int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                 int dtype, int block_size, const int32_t *blocks_host, int num_blocks,
                                 int num_ctas, int kernel_choice, sa_stream_t stream);

/*
 * Run-time seed selection: the middle seed blocks of every (row, KV head) pair are chosen by
 * scoring the K cache against the current query instead of taking fixed positions.  All three
 * steps stay on the device; the block list never visits the host.
 * Replaces _score_tensor_for_runtime_selector and select_seed_blocks_by_profile
 * (seed_selectors.py:274-396) for the selectors that need only q and K:
 *   SA_SELECT_QK_BLOCK_MAX  score = max over the block's tokens of q.k   ("qk_block_max")
 *   SA_SELECT_BLOCK_MEAN    score = q . mean key of the block            ("block_mean_proxy")
 *
 * sa_block_scores: scores[batch, q_heads, ceil(kv_len / block_size)] f32 (device), one score
 *   per query head as in the reference; blocks without valid tokens get -inf.  bf16/fp16.
 * sa_seed_list_length: entries per pair of the lists below: min(blocks of the cache,
 *   sink + recent (de-duplicated) + middle).
 * sa_select_seed_blocks: blocks_out[batch * kv_heads, list_length] int32 (device), ascending.
 *   A pair's block score is the maximum over the query heads that share the KV head; sink and
 *   recent blocks are always kept; the best `middle_seed_blocks` other blocks join them (ties:
 *   lower index), the policy's fixed middle blocks filling up if too few blocks have a score.
 * sa_seed_plan_create_device: seed-only decode plan that reads each pair's block list from
 *   `blocks_dev` (as written by sa_select_seed_blocks) at run time; includes_last_block != 0
 *   says that every list ends with the cache's last block (true whenever recent_blocks >= 1),
 *   which is how a partly filled last block is accounted for.  Entries outside the cache are
 *   skipped and reported as SA_DEV_BAD_PAGE.
 */
enum sa_block_selector { SA_SELECT_QK_BLOCK_MAX = 0, SA_SELECT_BLOCK_MEAN = 1 };
SA_API int sa_block_scores(const void *q, const void *k, float *scores, const void *seq_lens, int lens_dtype,
                           int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                           int64_t q_stride_b, int64_t q_stride_h,
                           int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                           int dtype, int block_size, int selector, sa_stream_t stream);
SA_API int sa_seed_list_length(int64_t kv_len, int block_size, int sink_blocks, int recent_blocks,
                               int middle_seed_blocks);
SA_API int sa_select_seed_blocks(const float *scores, int32_t *blocks_out, int batch, int q_heads, int kv_heads,
                                 int64_t kv_len, int block_size, int sink_blocks, int recent_blocks,
                                 int middle_seed_blocks, int block_order, sa_stream_t stream);
SA_API sa_plan_t *sa_seed_plan_create_device(const void *q, const void *k, const void *v, void *out,
                                             void *workspace, size_t workspace_bytes,
                                             int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                                             int64_t q_stride_b, int64_t q_stride_h,
                                             int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                             int dtype, int block_size, const int32_t *blocks_dev,
                                             int blocks_per_pair, int includes_last_block,
                                             int num_ctas, int kernel_choice);

/*
 * Exact merge of split states: states [num_parts, rows, D+2] f32 (layout of
 * SA_OUT_STATE) -> out [rows, D] in out_dtype.  Used after the cross-GPU
 * gather of context-parallel decode.  Same arithmetic as
 * _paged_exact_splitk_merge_kernel (kernels/paged_exact_triton.py:144-186)
 * and exact_merge_warp_out (transposed_gqa_exact_sources.py:1460-1522).
 */
SA_API int sa_merge_states(const float *states, int num_parts, int64_t rows, int head_dim,
                           void *out, int out_dtype, sa_stream_t stream);

/*
 * Context-parallel exchange fused with the merge (no counterpart in the reference, which has no
 * multi-GPU decode; the merge arithmetic is that of core/ring_attention.py:254-274).
 * Every rank owns one exchange buffer of sa_cp_exchange_bytes() bytes, zero-filled once, that
 * all ranks can address (peer-mapped / symmetric memory); peer_buffers is a HOST array with the
 * address of every rank's buffer as seen from this GPU (index = rank).  One call per decode step
 * on every rank, with the same step number (1, 2, 3, ...): the kernel stores local_state
 * [rows, D+2] into every rank's buffer with plain peer stores, raises this rank's flag there,
 * waits (at most the wait limit, 2 s by default, then SA_DEV_PIPELINE_TIMEOUT in the buffer's status word) for all ranks'
 * flags and writes the merged out [rows, D].  Buffers are double-buffered by step parity.
 */
#define SA_CP_MAX_WORLD 16
SA_API size_t sa_cp_exchange_bytes(int world_size, int64_t rows, int head_dim);
SA_API int sa_cp_exchange_merge(const float *local_state, const uint64_t *peer_buffers, int world_size, int rank,
                                uint32_t step, int64_t rows, int head_dim, void *out, int out_dtype,
                                sa_stream_t stream);
/* Synchronise and return (then clear) the status bits of an exchange buffer. */
SA_API int sa_cp_exchange_status(void *exchange_buffer, int world_size, int64_t rows, int head_dim,
                                 sa_stream_t stream);

/*
 * Context-parallel decode in ONE launch per step (no counterpart in the reference): the shard's
 * exact decode, the state exchange and the cross-rank merge fused.  The CTA that completes a
 * (row, KV head) pair on this rank stores the pair's state rows into every rank's exchange buffer
 * (plain peer stores; every 64-bit word carries the step number, so the data is its own flag),
 * waits (at most the plan's wait limit, 2 s by default, then SA_DEV_PIPELINE_TIMEOUT in the
 * workspace status word) for the same pair from all ranks and writes
 * the merged rows of out [batch, q_heads, D].  Up to 8 ranks; bf16/fp16, head_dim 64/128 (the
 * streaming kernel); uniform shard length.  Each rank's exchange buffer has
 * sa_cp_fused_bytes() bytes, is zero-filled once and addressable by all ranks; peer_buffers is a
 * HOST array of its address on every rank (index = rank).  Every sa_plan_run() of the returned
 * plan is one step; all ranks must run their plans the same number of times.
 */
SA_API size_t sa_cp_fused_bytes(int world_size, int batch, int q_heads, int kv_heads, int head_dim);
SA_API sa_plan_t *sa_cp_fused_plan_create(const void *q, const void *k, const void *v, void *out,
                                          void *workspace, size_t workspace_bytes,
                                          int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                                          int64_t q_stride_b, int64_t q_stride_h,
                                          int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                          int dtype, int num_ctas,
                                          const uint64_t *peer_buffers, int world_size, int rank);

/*
 * Bound plans: validate once, keep the prepared launch (tensor maps, geometry),
 * run many times with no per-call setup - what ExactDecodePlan.run /
 * PagedExactDecodePlan.run do in the reference
 * (transposed_gqa_exact.py:381-430, paged.py:490-538).  The create functions take
 * the same arguments as the one-shot calls (without the stream) and return NULL
 * on error.  A plan holds pointers, not ownership; the buffers must outlive it.
 */
SA_API sa_plan_t *sa_exact_plan_create(const void *q, const void *k, const void *v, void *out,
                                       void *workspace, size_t workspace_bytes,
                                       const void *seq_lens, int lens_dtype,
                                       int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                                       int64_t q_stride_b, int64_t q_stride_h,
                                       int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                       int dtype, int out_mode, int num_ctas, int kernel_choice);

SA_API sa_plan_t *sa_paged_plan_create(const void *q, const void *k_pages, const void *v_pages,
                                       const void *page_table, const void *seq_lens, void *out,
                                       void *workspace, size_t workspace_bytes, int32_t *trace,
                                       int batch, int q_heads, int kv_heads, int head_dim,
                                       int page_size, int max_pages_per_request, int64_t num_pages,
                                       int layout, int dtype, int table_dtype, int lens_dtype,
                                       int out_mode, int num_ctas, int kernel_choice);

SA_API sa_plan_t *sa_seed_plan_create(const void *q, const void *k, const void *v, void *out,
                                      void *workspace, size_t workspace_bytes,
                                      int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                                      int64_t q_stride_b, int64_t q_stride_h,
                                      int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                      int dtype, int block_size, const int32_t *blocks_host, int num_blocks,
                                      int num_ctas, int kernel_choice);

SA_API int sa_plan_run(const sa_plan_t *plan, sa_stream_t stream);
/* 1 = TMA/tensor-core streaming kernel, 2 = generic CUDA-core kernel. */
SA_API int sa_plan_kernel(const sa_plan_t *plan);
/* CTAs the plan launches and kernels enqueued per run. */
SA_API int sa_plan_num_ctas(const sa_plan_t *plan);
SA_API int sa_plan_launches(const sa_plan_t *plan);
SA_API void sa_plan_destroy(sa_plan_t *plan);

/*
 * Row subset of a bound plan: compute only the batch rows listed in the DEVICE array `rows`
 * (index_dtype int32/int64, num_rows entries read at run time; entries outside [0, batch) are
 * ignored, duplicates are harmless) and leave the output rows of every other batch row
 * untouched.  rows = NULL restores "every row".  Replaces the row_indices argument of
 * exact_decode_attention_rows_triton_forward_out_bhnd (kernels/gate0_exact_refresh_triton.py:
 * 251-259, 266-344: "only selected rows are overwritten").  Not for fused context-parallel plans.
 */
SA_API int sa_plan_set_rows(sa_plan_t *plan, const void *rows, int index_dtype, int num_rows);

/*
 * Limit of the bounded device-side waits (TMA copy barriers, split states in flight between
 * the CTAs of a launch, a peer rank's words in the context-parallel exchange).  A wait that
 * runs out sets SA_DEV_PIPELINE_TIMEOUT in the status word and the kernel returns; nothing
 * hangs or traps.  Default 2 s.  sa_set_wait_limit_ns sets the process-wide default that
 * plans created afterwards, the one-shot calls and sa_cp_exchange_merge use;
 * sa_plan_set_wait_limit_ns changes one plan.  No counterpart in the reference, whose
 * kernels do not wait on each other.
 */
SA_API int sa_set_wait_limit_ns(uint64_t limit_ns);
SA_API int sa_plan_set_wait_limit_ns(sa_plan_t *plan, uint64_t limit_ns);

/* ---- KV-cache update: the step before each decode call ------------------------------------
 * Writes the current token's K/V row of every (row, KV head) into the cache at the row's
 * position, optionally after the rotary embedding, and optionally rotates the query as well:
 *     x' = x * cos + rotate_half(x) * sin,   rotate_half(x) = concat(-x[D/2:], x[:D/2])
 * evaluated in the cache dtype with every product and the sum rounded to that dtype, i.e. the
 * bits of the same expression on torch tensors.  Replaces the reference's
 * `_apply_qwen_rope` + `copy_` pair (benchmarks/profile_seed_only_fused_rope_parity.py:24-30,
 * 97-102), its append kernel (benchmarks/profile_kv_cache_update_floor.py:46-75) and the
 * RoPE + append prologue of its fused seed kernel (kernels/gate0_seed_only_triton.py:731-770).
 *
 *   k_new, v_new   [batch, kv_heads, D] rows, strides new_stride_b / new_stride_h (elements)
 *   positions      device int32/int64: one entry (all rows share it, like the reference's
 *                  cache_position) or one per row; the token index written
 *   lens_out       optional device array [batch] (same integer type): receives position + 1;
 *                  may be the per-row `positions` array itself (in-place length advance)
 *   cos, sin       optional [batch or 1, D] in the cache dtype (rope_stride_b = 0: shared row);
 *                  NULL = plain append
 *   q_in / q_out   optional [batch, q_heads, D] rows (own strides): rotated query; must not alias
 *   status         optional device int32: SA_DEV_BAD_POSITION / SA_DEV_BAD_PAGE are OR-ed in when a
 *                  row's position or page id is out of range (that row is skipped, never written)
 */
#define SA_DEV_BAD_POSITION 4
SA_API int sa_append_kv(const void *k_new, const void *v_new, void *k_cache, void *v_cache,
                        const void *positions, int pos_dtype, int num_positions, void *lens_out,
                        const void *cos, const void *sin, int64_t rope_stride_b,
                        const void *q_in, void *q_out, int q_heads,
                        int64_t q_in_stride_b, int64_t q_in_stride_h, int64_t q_out_stride_b, int64_t q_out_stride_h,
                        int batch, int kv_heads, int head_dim, int64_t kv_len,
                        int64_t new_stride_b, int64_t new_stride_h,
                        int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                        int dtype, int *status, sa_stream_t stream);
/* Same for a paged cache: the row goes to slot position % page_size of page
 * page_table[b][position / page_size], which the caller's allocator must have assigned. */
SA_API int sa_paged_append_kv(const void *k_new, const void *v_new, void *k_pages, void *v_pages,
                              const void *page_table, int table_dtype,
                              const void *positions, int pos_dtype, int num_positions, void *lens_out,
                              const void *cos, const void *sin, int64_t rope_stride_b,
                              const void *q_in, void *q_out, int q_heads,
                              int64_t q_in_stride_b, int64_t q_in_stride_h, int64_t q_out_stride_b,
                              int64_t q_out_stride_h,
                              int batch, int kv_heads, int head_dim, int page_size, int max_pages,
                              int64_t num_pages, int layout, int64_t new_stride_b, int64_t new_stride_h,
                              int dtype, int *status, sa_stream_t stream);

/* ---- Output projection: the step after each decode call ----------------------------------
 * out[b, n] = sum_k x[b, k] * weight[n, k] (+ bias[n]) for the few rows of a decode step, fp32
 * accumulation, result in the input dtype (bf16/fp16).  Replaces qwen_o_proj_triton_forward
 * (kernels/qwen_o_proj_triton.py:77-145; kernel :25-74), i.e. F.linear on [batch, 1, hidden].
 *   x       [batch, in_features], rows x_stride_b elements apart (the attention output)
 *   weight  [out_features, in_features] contiguous (PyTorch's layout);  bias [out_features] or NULL
 *   out     [batch, out_features] contiguous
 * in_features and x_stride_b must be multiples of 8, x and weight 16-byte aligned.
 * prefetch_weights != 0: the kernel may start reading weight (never x) before earlier work of
 * `stream` has finished, which hides the weight stream behind the tail of the attention kernel;
 * pass 0 if the weights are written by work that was enqueued on `stream` just before. */
SA_API int sa_o_proj(const void *x, const void *weight, const void *bias, void *out,
                     int batch, int in_features, int out_features, int64_t x_stride_b,
                     int dtype, int prefetch_weights, sa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* STREAMATTN_B200_H_ */
