/*
 * aptserve_b200.h -- C ABI of the B200 (sm_100a) hybrid-cache data path.
 *
 * Every entry point replaces one operator the Apt-Serve reference reaches from
 * Python on its decode / cache-write hot path.  File:line citations name the
 * reference interface each one stands in for (paths inside the reference
 * project, under additional_designs/):
 *   mc.cu  = mixed_cache_kernels/mixed_cache.cu
 *   fa.py  = attention/backends/aptserve_flash_attn.py
 *   opt.py = model_executor/models/aptserve_opt.py
 *   lin.py = model_executor/layers/aptserve_linear.py
 *
 * Conventions
 *  - plain pointers and sizes only; all data pointers are DEVICE pointers unless
 *    a parameter says "host";
 *  - strides are in ELEMENTS of the payload dtype;
 *  - index tensors are int64 (slot mappings, index lists) or int32 (block tables,
 *    sequence lengths), exactly as the reference's model runner builds them;
 *  - every call enqueues on `stream` (a cudaStream_t passed as void*) of the
 *    CURRENT device and returns without synchronising;
 *  - nothing is allocated or freed for the caller and no pointer is retained
 *    after return;
 *  - the return value is an aps_status; no C++ exception crosses the boundary;
 *    aps_last_error() gives a human-readable message for the calling thread;
 *  - ONE calling thread per process, one call at a time (the reference's worker is
 *    single-threaded Python, one process per GPU): per-device launch geometry, the
 *    table of encoded tensor maps, the address of the built-in scratch and the
 *    profile-event hook are plain process- or thread-local statics without locks.
 *    Different processes on different GPUs are independent;
 *  - the library reads no environment variable.
 */
#ifndef APTSERVE_B200_H_
#define APTSERVE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum aps_status {
  APS_OK = 0,
  APS_ERR_NULL_POINTER = 1,  /* a required pointer is NULL                        */
  APS_ERR_MISALIGNED = 2,    /* pointer / stride not aligned as the op requires    */
  APS_ERR_DTYPE = 3,         /* dtype enum not supported by this op                */
  APS_ERR_SHAPE = 4,         /* negative / inconsistent sizes or strides           */
  APS_ERR_UNSUPPORTED = 5,   /* head size / block size / hidden size not supported */
  APS_ERR_WORKSPACE = 6,     /* workspace NULL, misaligned or too small            */
  APS_ERR_CUDA = 7,          /* a CUDA runtime / driver call failed                */
  APS_ERR_DEVICE = 8         /* device-side status word reported a failure         */
} aps_status;

typedef enum aps_dtype {
  APS_F32 = 0,
  APS_F16 = 1,
  APS_BF16 = 2
} aps_dtype;

/* Message describing the last non-zero status returned on this thread. */
const char* aps_last_error(void);

/* Library version string, e.g. "aptserve_b200 0.1 (sm_100a)". */
const char* aps_version(void);

/* ------------------------------------------------------------------------ */
/* Paged cache writes (bit-exact data movement, HBM-bound)                   */
/* ------------------------------------------------------------------------ */

/*
 * Replaces vllm._custom_ops.reshape_and_cache_flash as called at fa.py:338-345,
 * fa.py:348-355 and fa.py:378-385:
 *   key_cache[slot / BS, slot % BS, :, :] = key[t]   (same for value), slot < 0 skipped.
 * key/value: [T, H, D] with row strides key_stride / value_stride;
 * caches: [NB, BS, H, D], block stride block_stride, [BS, H, D] contiguous inside.
 */
int aps_reshape_and_cache(const void* key, const void* value, void* key_cache,
                          void* value_cache, const int64_t* slot_mapping,
                          int64_t num_tokens, int num_heads, int head_size,
                          int block_size, int64_t key_stride, int64_t value_stride,
                          int64_t block_stride, int dtype, void* stream);

/*
 * Replaces mixed_cache_ops.hidden_to_cache (mc.cu:119-147, kernel mc.cu:31-53;
 * called at opt.py:108-109): for i in [0, n):
 *   slot = slot_mapping[target_slot_idx[i]]; if slot >= 0:
 *   paged_cache[slot * slot_stride + (0..hidden_size)] = hidden[src_idx[i], :]
 * slot_stride is paged_cache.stride(2) of the [2, NB, BS, H, D] tensor.
 */
int aps_hidden_to_cache(const void* hidden, void* paged_cache,
                        const int64_t* slot_mapping, const int64_t* src_idx,
                        const int64_t* target_slot_idx, int64_t n, int hidden_size,
                        int64_t hidden_stride, int64_t slot_stride, int dtype,
                        void* stream);

/*
 * Replaces mixed_cache_ops.cache_to_hidden (mc.cu:150-176, kernel mc.cu:6-28;
 * called at opt.py:120-121): for i in [0, n): t = dst_idx[i];
 *   slot = slot_mapping[t]; if slot >= 0: hidden[t, :] = paged_cache[slot * slot_stride + ...]
 */
int aps_cache_to_hidden(void* hidden, const void* paged_cache,
                        const int64_t* slot_mapping, const int64_t* dst_idx, int64_t n,
                        int hidden_size, int64_t hidden_stride, int64_t slot_stride,
                        int dtype, void* stream);

/*
 * Replaces mixed_cache_ops.mixed_kv_to_cache (mc.cu:179-230, kernel mc.cu:56-116;
 * called at fa.py:363-373):
 *   b in [0, n_kv):  tok = kv_cache_use_tot[b], slot = slot_mapping[tok]:
 *                    key/value[tok] -> k_cache/v_cache AND shared_k/shared_v at slot
 *   j in [0, n_hidden): tok = hidden_cache_use_tot[j], slot = slot_mapping_shared[j]:
 *                    key/value[tok] -> shared_k/shared_v at slot
 * (j is the hidden token's ordinal; the reference's `blockIdx.x % (2*n_kv)` at
 * mc.cu:88 equals it only while n_hidden <= 2*n_kv.)
 */
int aps_mixed_kv_to_cache(const void* key, const void* value, void* k_cache,
                          void* v_cache, void* shared_k_cache, void* shared_v_cache,
                          const int64_t* slot_mapping,
                          const int64_t* slot_mapping_shared,
                          const int64_t* kv_cache_use_tot,
                          const int64_t* hidden_cache_use_tot, int64_t n_kv,
                          int64_t n_hidden, int num_heads, int head_size,
                          int block_size, int64_t key_stride, int64_t value_stride,
                          int64_t block_stride, int64_t shared_block_stride, int dtype,
                          void* stream);

/*
 * Prefill cache write in one launch: replaces the pair of calls a prefill batch with
 * hidden-designated prompts makes -- mixed_cache_ops.hidden_to_cache for the hidden-designated
 * token rows (opt.py:108-109) and reshape_and_cache_flash on the index-selected
 * key[kv_cache_use_tot] / value[kv_cache_use_tot] (fa.py:347-355):
 *   i in [0, n_kv):     t = kv_rows[i];     key/value[t] -> K / V plane at slot_mapping[t]
 *   j in [0, n_hidden): t = hidden_rows[j]; hidden[t, :]  -> flat hidden row slot_mapping[t]
 * kv_rows / hidden_rows are the metadata's kv_cache_use_tot / hidden_cache_use_input.
 * No gathered copy of key / value is made.
 */
int aps_prefill_cache_write(const void* key, const void* value, const void* hidden,
                            void* key_cache, void* value_cache, void* hidden_cache,
                            const int64_t* slot_mapping, const int64_t* kv_rows, int64_t n_kv,
                            const int64_t* hidden_rows, int64_t n_hidden, int num_heads,
                            int head_size, int hidden_size, int block_size, int64_t key_stride,
                            int64_t value_stride, int64_t hidden_stride, int64_t block_stride,
                            int64_t slot_stride, int dtype, void* stream);

/*
 * Replaces vllm._custom_ops.swap_blocks as called at fa.py:44-56 (once per layer and plane):
 *   dst[d] = src[s] for every row (s, d) of the HOST array pairs_host [num_pairs, 2],
 * src / dst being one plane [num_blocks, BS, H, D] of a GPU cache or of the pinned CPU
 * cache.  kind: 0 = host to device (swap in), 1 = device to host (swap out), 2 = device to
 * device.  Copies are enqueued on `stream` from a native loop; runs of pairs whose source and
 * destination blocks are both consecutive become one copy.  copies_issued (may be NULL)
 * receives the number of copies enqueued.
 */
int aps_swap_blocks(const void* src, void* dst, const int64_t* pairs_host, int64_t num_pairs,
                    int64_t block_bytes, int64_t src_block_stride_bytes, int64_t dst_block_stride_bytes,
                    int64_t src_num_blocks, int64_t dst_num_blocks, int kind, int64_t* copies_issued,
                    void* stream);

/*
 * Replaces vllm._custom_ops.copy_blocks as called at fa.py:58-65:
 * for every layer l and every row (src, dst) of block_mapping [num_pairs, 2]:
 *   key_caches[l][dst] = key_caches[l][src]; value_caches[l][dst] = value_caches[l][src].
 * key_cache_ptrs / value_cache_ptrs are HOST arrays of num_layers device
 * pointers; block_bytes is the size of one block of one plane.
 */
int aps_copy_blocks(void* const* key_cache_ptrs, void* const* value_cache_ptrs,
                    int num_layers, const int64_t* block_mapping, int64_t num_pairs,
                    int64_t block_bytes, void* stream);

/* ------------------------------------------------------------------------ */
/* Decode attention                                                          */
/* ------------------------------------------------------------------------ */

/*
 * Bytes of scratch the two attention calls below need for a batch of `batch`
 * requests whose block tables are `max_blocks_per_seq` wide.  The caller
 * allocates it (256-byte aligned) and may reuse it across calls on one stream.
 */
size_t aps_attention_workspace_bytes(int batch, int max_blocks_per_seq,
                                     int block_size, int num_heads, int head_size);

/*
 * Replaces vllm_flash_attn.flash_attn_with_kvcache as called at fa.py:452-461
 * (decode batch, all requests K/V-cached):
 *   out[r, h, :] = softmax(scale * q[r, h] . K_r[:, h]) @ V_r[:, h]
 * over the first seq_lens[r] tokens found through block_tables[r].
 * query/out: [B, H*D] with row strides; caches [NB, BS, H, D];
 * block_tables int32 [B, max_blocks_per_seq]; seq_lens int32 [B].
 */
int aps_paged_decode_attention(void* out, const void* query, const void* key_cache,
                               const void* value_cache, const int32_t* block_tables,
                               const int32_t* seq_lens, int batch,
                               int max_blocks_per_seq, int num_heads, int head_size,
                               int block_size, int64_t query_stride,
                               int64_t out_stride, int64_t block_stride, float scale,
                               void* workspace, size_t workspace_bytes, int dtype,
                               void* stream);

/*
 * aps_paged_decode_attention for callers that cannot allocate device memory.
 * This one has no counterpart in the reference.  Same arguments and result as
 * aps_paged_decode_attention, minus the workspace: the scratch is a 32 MiB array
 * built into the library's device image (each GPU that loads the library holds
 * those 32 MiB until the process exits).  It serves hosts that bind this ABI
 * without an allocator of their own -- a serving worker whose cache engine has
 * already claimed all free HBM for K/V blocks, or a C / Go / Java host with no
 * device-memory pool, for which a cudaMalloc per step would also stall the device.
 *  - No cudaMalloc, cudaFree or allocating library call is made.
 *  - A batch whose scratch need (aps_attention_workspace_bytes of its shape)
 *    exceeds 32 MiB is rejected with APS_ERR_WORKSPACE; e.g. 64 requests x 2048
 *    tokens at 40 heads x 128 need about 23 MiB and fit, 256 such requests do not.
 *  - Every call looks up the array's device address (cudaGetSymbolAddress, with
 *    the calling thread's device current) and keeps nothing between calls, so a host
 *    that tears its CUDA context down and builds a new one is served correctly.
 *    The very first lookup on a device loads the library's device image: make a
 *    first call on each device before any stream capture begins.
 *  - All calls share the one array.  Everything a call reads from it is written
 *    earlier in the same call (its first kernel resets the work counter, the list
 *    sizes and the status word), so stale contents are harmless; but two calls
 *    that overlap on the GPU (different streams, no ordering) race on it.
 */
int aps_paged_decode_attention_static(void* out, const void* query, const void* key_cache,
                                      const void* value_cache, const int32_t* block_tables,
                                      const int32_t* seq_lens, int batch,
                                      int max_blocks_per_seq, int num_heads, int head_size,
                                      int block_size, int64_t query_stride,
                                      int64_t out_stride, int64_t block_stride, float scale,
                                      int dtype, void* stream);

/*
 * Hybrid decode attention: one call for the decode branch of
 * OPTAttention.forward with hidden-cached requests (opt.py:111-124: gather of
 * cached hidden rows, K/V re-projection lin.py:123-130) followed by the cache
 * write + paged attention of fa.py:356-387 and fa.py:462-473 -- without the
 * hidden_holder buffer, the [N_tot, 2HD] K/V tensor or the shared cache.
 *
 *   cache_type[r] == 0: K/V rows come from key_cache/value_cache through
 *                       block_tables[r] (as aps_paged_decode_attention);
 *   cache_type[r] != 0: hidden rows X_r come from the flat rows of hidden_cache
 *                       (row id = block_tables[r][t / BS] * BS + t % BS, row
 *                       stride hidden_row_stride, first hidden_size elements);
 *                       K = X_r W_k^T + b_k, V = X_r W_v^T + b_v on the tensor
 *                       cores, fp32 accumulation, then the same softmax.
 * w_k / w_v: [H*D, hidden_size] row-major with row stride w_stride (the K and V
 * thirds of the fused QKV weight, lin.py:123-125); b_k / b_v: [H*D] or NULL.
 * num_hidden_rows is the number of addressable rows of hidden_cache
 * (2*NB*BS for the reference layout).  fp16 / bf16 with head_size 128, 64 or 32 and
 * num_heads * head_size a multiple of 128 use the tcgen05 path (two heads of 64 or four
 * of 32 share one accumulator tile); other supported combinations (fp32, other head
 * counts) use a CUDA-core re-projection.
 * key_cache / value_cache may both be NULL for a batch without K/V-cached requests;
 * if such a batch does hold K/V-cached requests their output rows are zero and the
 * status word (aps_attention_status) reads 8.
 */
int aps_hybrid_decode_attention(void* out, const void* query, const void* key_cache,
                                const void* value_cache, const void* hidden_cache,
                                const void* w_k, const void* b_k, const void* w_v,
                                const void* b_v, const int32_t* block_tables,
                                const int32_t* seq_lens, const int32_t* cache_type,
                                int batch, int max_blocks_per_seq, int num_heads,
                                int head_size, int hidden_size, int block_size,
                                int64_t query_stride, int64_t out_stride,
                                int64_t block_stride, int64_t hidden_row_stride,
                                int64_t num_hidden_rows, int64_t w_stride, float scale,
                                void* workspace, size_t workspace_bytes, int dtype,
                                void* stream);

/*
 * The K/V re-projection on its own (opt.py:123 -> lin.py:123-130):
 *   kv[t, 0:HD] = X[t] W_k^T + b_k ; kv[t, HD:2HD] = X[t] W_v^T + b_v ,  t in [0, n_rows)
 * Same tensor-core main loop as the hybrid attention; fp16 / bf16, head_size 128, 64 or
 * 32 with num_heads * head_size a multiple of 128.
 *   block_ids == NULL : X[t] is row t of x (the dense hidden_holder of opt.py:112-121);
 *   block_ids != NULL : X[t] is row block_ids[t / 16] * 16 + t % 16 of x, i.e. x is a
 *                       paged hidden cache read in 16-row blocks (int32 ids).
 * x: rows of x_row_stride elements, num_x_rows addressable rows; kv: [n_rows, 2*HD]
 * with row stride kv_stride.  status_word (device int, zeroed by the caller, may be
 * NULL) receives a non-zero code if a bounded device-side wait ran out.
 */
int aps_kv_reprojection(void* kv, const void* x, const int32_t* block_ids, int64_t n_rows,
                        const void* w_k, const void* b_k, const void* w_v, const void* b_v,
                        int num_heads, int head_size, int hidden_size, int64_t x_row_stride,
                        int64_t num_x_rows, int64_t w_stride, int64_t kv_stride, int dtype,
                        int* status_word, void* stream);

/*
 * One decode layer-step in one call: everything between the projections and o_proj
 * of OPTAttention.forward's decode branch (opt.py:99-134 with fa.py:331-387,
 * 449-475).  Enqueues, in this order,
 *   1. the new token's cache writes, addressed from block_tables / seq_lens /
 *      cache_type (position seq_lens[r] - 1): hidden_states[r] -> hidden cache row for
 *      hidden-cached requests (hidden_to_cache, opt.py:108-109), new_key[r] /
 *      new_value[r] -> K/V planes for K/V-cached requests (the private-cache half of
 *      mixed_kv_to_cache, fa.py:363-373, or reshape_and_cache_flash, fa.py:338-345);
 *   2. aps_hybrid_decode_attention over the batch.
 * hidden_states [B, hidden_size], new_key / new_value [B, H*D] (rows of the other
 * cache type are ignored; a NULL pointer skips that kind of write), every pointer
 * and row 16-byte aligned.  All other arguments as in aps_hybrid_decode_attention.
 */
int aps_decode_layer_step(void* out, const void* query, const void* hidden_states,
                          const void* new_key, const void* new_value, void* key_cache,
                          void* value_cache, void* hidden_cache, const void* w_k,
                          const void* b_k, const void* w_v, const void* b_v,
                          const int32_t* block_tables, const int32_t* seq_lens,
                          const int32_t* cache_type, int batch, int max_blocks_per_seq,
                          int num_heads, int head_size, int hidden_size, int block_size,
                          int64_t query_stride, int64_t out_stride, int64_t hidden_states_stride,
                          int64_t new_key_stride, int64_t new_value_stride, int64_t block_stride,
                          int64_t hidden_row_stride, int64_t num_hidden_rows, int64_t w_stride,
                          float scale, void* workspace, size_t workspace_bytes, int dtype,
                          void* stream);

/*
 * Reads the status word the attention kernels keep in `workspace` for the last call
 * that used it.  0 = fine.  1..7 = a bounded device-side wait of the re-projection
 * kernel ran out (the kernel returned early; the call's whole output was filled with
 * NaN).  8 = the batch held K/V-cached requests but no K/V cache was passed (their
 * output rows are zero).  Synchronises `stream`: call it where a synchronisation is
 * cheap, e.g. once per engine step next to the sampler's device-to-host copy.
 */
int aps_attention_status(const void* workspace, int* host_status, void* stream);

/*
 * SM clock cycles CTA 0 of the tensor-core re-projection kernel spent in the last hybrid
 * call that used `workspace` (two clock reads per launch, always recorded).  Against the
 * cycles the tensor cores need for the call's tiles (512 per 64-element slab of a 256 x 256
 * tile pair) this is the kernel's tensor-pipe utilisation, independent of sampled clocks.
 * Synchronises `stream`.  No reference counterpart.
 */
int aps_reprojection_cycles(const void* workspace, unsigned long long* host_cycles, void* stream);

/*
 * Status of the bulk-copy cache writes on the current device: 0, or 1 once a bounded
 * wait on a bulk load ran out (the launch then stopped copying).  Synchronises `stream`.
 */
int aps_cache_ops_status(int* host_status, void* stream);

/*
 * Test aid for the status handling (no counterpart in the reference).  `workspace` must
 * have been used by an attention call of the given shape.  One thread waits on an
 * mbarrier that nothing arrives on, gives up after budget_cycles clock cycles (1 .. 1e8,
 * i.e. at most ~0.1 s) and records code 7 in the workspace's status word, exactly as the
 * bounded waits of the re-projection kernel do; then the attention's combine step runs
 * again over the workspace and, seeing the code, fills `out` [batch, H*D] with NaN.
 * Nothing hangs or faults and the context stays usable.
 */
int aps_selftest_bounded_wait(void* workspace, size_t workspace_bytes, long long budget_cycles,
                              void* out, int batch, int max_blocks_per_seq, int num_heads,
                              int head_size, int block_size, int64_t out_stride, int dtype,
                              void* stream);

/* ------------------------------------------------------------------------ */
/* Index tensors                                                             */
/* ------------------------------------------------------------------------ */

/*
 * Replaces the decode branch of ModelRunner._prepare_model_input
 * (additional_designs/worker/aptserve_model_runner.py:515-564 per-request loop,
 * :613-648 mask-to-index conversion): expands the block tables on the device into
 * the eight int64 index tensors of a decode batch, instead of building them with a
 * Python loop over every cached position of every hidden-cached request and copying
 * them to the device each step.
 *   block_tables         int32 [B, max_blocks]  private tables (hidden requests: V-plane ids for odd blocks)
 *   block_tables_shared  int32 [B, max_blocks]  shared tables of hidden requests (rows of K/V requests unused)
 *   seq_lens int32 [B] (>= 1, includes the token being decoded), cache_type int32 [B]
 * Outputs (sizes as in the reference: N_tot = sum over hidden requests of S_r + number of
 * K/V requests, N_h = sum over hidden requests of S_r, n_kv, n_h = request counts):
 *   slot_mapping [N_tot], slot_mapping_shared [N_h], hidden_cache_use_tot [N_h],
 *   kv_cache_use_tot [n_kv], hidden_holder_upd [B], hidden_holder_pull [N_tot - B],
 *   hidden_cache_store_tot [n_h], hidden_cache_use_input [n_h].
 * num_tot_tokens / num_hidden_tokens are the caller's N_tot / N_h (the host knows them from
 * the sequence lengths; a length below 1 counts as 1); n_kv = N_tot - N_h and n_h = B - n_kv
 * follow.  An output that is empty for these counts may be NULL.  The kernels recompute the
 * four counts from the device-side seq_lens / cache_type: if they differ from the caller's,
 * NOTHING is written (the outputs keep their previous contents), and no store ever goes past
 * a tensor's capacity.  counts (device int64[4], may be NULL) receives N_tot, N_h, n_kv, n_h
 * as computed on the device, so a caller can detect the mismatch.
 * scratch: aps_decode_metadata_scratch_bytes(B) bytes of device memory.
 */
size_t aps_decode_metadata_scratch_bytes(int batch);
int aps_expand_decode_metadata(const int32_t* block_tables, const int32_t* block_tables_shared,
                               const int32_t* seq_lens, const int32_t* cache_type, int batch,
                               int max_blocks_per_seq, int block_size, int64_t* slot_mapping,
                               int64_t* slot_mapping_shared, int64_t* hidden_cache_use_tot,
                               int64_t* kv_cache_use_tot, int64_t* hidden_holder_upd,
                               int64_t* hidden_holder_pull, int64_t* hidden_cache_store_tot,
                               int64_t* hidden_cache_use_input, int64_t num_tot_tokens,
                               int64_t num_hidden_tokens, int64_t* counts, void* scratch,
                               size_t scratch_bytes, void* stream);

/*
 * Timing hook for benchmarks (no counterpart in the reference, whose kernels are
 * timed with commented-out torch.cuda.synchronize() calls, fa.py:374-387):
 * while set (a thread-local, unsynchronised hook), the attention calls of THIS THREAD record `start_event` just before
 * and `stop_event` just after the launch of the K/V streaming kernel (which = 0)
 * or of the re-projection kernel (which = 1), on the stream of the call.  Events
 * are cudaEvent_t handles owned by the caller; pass NULL, NULL to switch off.
 */
int aps_set_profile_events(int which, void* start_event, void* stop_event);

/*
 * Hidden-path decode attention with the projections absorbed (no counterpart in the
 * reference, which re-projects every cached hidden row, opt.py:111-124).  For a hidden
 * request and head h, q.(W_k,h x_t + b_k) = (W_k,h^T q).x_t + const and
 * sum_t p_t (W_v,h x_t + b_v) = W_v,h (sum_t p_t x_t) + b_v, so the cached hidden rows can
 * be attended directly.  The caller folds `absorbed_query[h][i][:] = scale * log2(e) *
 * W_k,h^T q[req_rows[i]][h]` ([heads_padded, n_req, hidden], model dtype, heads padded with
 * zero rows to a multiple of 16: 16, 32, 48 or 80) with one batched GEMM; this call writes
 * `scores` (scratch: [tok_offset[n_req], heads_padded] fp32, tok_offset = prefix sums of the
 * hidden requests' clipped lengths), `probs` (scratch of the same shape in the model dtype:
 * the softmax of the scores over each request's tokens) and `z[h][i][:] = sum_t softmax_t(scores)[t][h] x_t`
 * ([heads_padded, n_req, hidden], model dtype); the caller unfolds out[h] = W_v,h z[h] + b_v
 * with a second batched GEMM.  `block_tables` / `seq_lens` are the whole batch's; `req_rows`
 * names the batch rows of the hidden requests.  fp16 / bf16, hidden_size % 512 == 0.
 */
int aps_absorbed_hidden_attention(void* z, float* scores, void* probs, const void* hidden_cache,
                                  const void* absorbed_query, const int32_t* block_tables,
                                  const int32_t* seq_lens, const int32_t* req_rows,
                                  const int64_t* tok_offset, int n_req, int max_blocks_per_seq,
                                  int block_size, int hidden_size, int heads_padded,
                                  int64_t hidden_row_stride, int64_t num_hidden_rows, int dtype,
                                  void* stream);

/*
 * Tensor-parallel exchange: the one collective of the path.  Replaces
 * vllm.distributed.tensor_model_parallel_all_reduce as RowParallelLinear.forward calls
 * it on the o_proj output of every layer (lin.py:827-829; the bias is added by the
 * caller after the reduce, lin.py:833-834).  One process per GPU; the communicator is
 * created on the calling thread's current CUDA device and wraps one NCCL communicator.
 * NCCL is resolved at run time from the libnccl.so.2 the process has loaded (or the
 * system's); if none is found every call returns APS_ERR_UNSUPPORTED.
 *
 *  aps_tp_unique_id   rank 0 fills `unique_id_out` (APS_TP_UNIQUE_ID_BYTES host bytes)
 *                     and hands the bytes to the other ranks over the host's own channel
 *                     (the reference has torch.distributed / Ray for that).
 *  aps_tp_init        collective over all ranks: every rank passes the same id, its
 *                     rank and the world size; blocks until all have joined.
 *  aps_tp_allreduce   in-place sum of `count` elements of `dtype` at `buffer` (device
 *                     memory), enqueued on `stream`; returns without synchronising.
 *  aps_tp_world_size  number of ranks of the communicator.
 *  aps_tp_destroy     releases the communicator (NULL is accepted).
 */
#define APS_TP_UNIQUE_ID_BYTES 128
int aps_tp_unique_id(void* unique_id_out);
int aps_tp_init(void** comm_out, const void* unique_id, int rank, int world_size);
int aps_tp_allreduce(void* comm, void* buffer, int64_t count, int dtype, void* stream);
int aps_tp_world_size(void* comm, int* world_size_out);
int aps_tp_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif /* APTSERVE_B200_H_ */
