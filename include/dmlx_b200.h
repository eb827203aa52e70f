/*
 * dmlx_b200.h — C-ABI of the B200-native continuous-batching decode path.
 *
 * Plain C99: fixed-width integers, opaque handles, caller-allocated out-arrays with explicit
 * capacities, no callbacks.  Bound from Zig with @cImport, from C/C++ directly and from Python
 * with ctypes.  Every entry point names the reference interface it stands in for (path within the
 * reference project : line).
 *
 * Conventions
 *  - Every function that can fail returns a b200_status; b200_last_error() gives a message for
 *    the calling thread's last failure.
 *  - A context (kv pool, model, scheduler ...) is single-owner and not thread-safe, like the
 *    reference's single engine thread.  One device and one calling thread per process: the library
 *    keeps per-process caches (matmul scratch, shared-memory opt-ins) for the first device a compute
 *    entry point runs on and refuses calls made with another device current (B200_ERR_UNSUPPORTED);
 *    all matmuls of a process share one split-K scratch, so they belong on one stream (or on streams
 *    ordered by events).  b200_qmm_static_scratch alone keeps its state per device.
 *  - Device pointers are plain `void*`/typed pointers to memory on the current CUDA device; streams
 *    are passed as `void*` (a cudaStream_t; NULL = the default stream).
 *  - Conditions detected inside a kernel (pool exhausted, bad index) are reported through an error
 *    word read after the step (b200_kv_error_word); kernels never trap.
 *  - There is no CPU fallback: compute entry points return B200_ERR_NO_DEVICE without a GPU.
 */
#ifndef DMLX_B200_H
#define DMLX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------ */
/* Status codes: the reference's Zig error set for this path, one to one.                      */
/* ------------------------------------------------------------------------------------------ */
typedef int32_t b200_status;
enum {
  B200_OK = 0,
  B200_ERR_INSUFFICIENT_BLOCKS = 1, /* src/kvcache/paged.zig:109,174; src/scheduler.zig:64 */
  B200_ERR_INVALID_BLOCK_ID = 2,    /* src/kvcache/paged.zig:168,269 */
  B200_ERR_PAGE_POOL_EXHAUSTED = 3, /* src/kvcache/paged.zig:427 */
  B200_ERR_INVALID_QUANT_BITS = 4,  /* src/kvcache/paged.zig:355 */
  B200_ERR_INVALID_BATCH_INDEX = 5, /* src/kvcache/paged.zig:904 */
  B200_ERR_INVALID_ARGUMENT = 6,
  B200_ERR_CUDA = 7,
  B200_ERR_NO_DEVICE = 8,
  B200_ERR_UNSUPPORTED = 9,         /* src/kvcache/interface.zig:119,136 (FilterNotSupported ...) */
  B200_ERR_CAPACITY = 10,           /* out-array too small / src/kvcache/quantized.zig:135 CacheOverflow */
  B200_ERR_DEVICE_FLAGGED = 11,     /* a kernel set the error word; see b200_kv_error_word */
  B200_ERR_CANCELLED = 12           /* src/engine/request_state.zig:118,182-189 (cancelled flag) */
};
const char* b200_status_name(b200_status s);
const char* b200_last_error(void);
/* Library version, and 1 if a CUDA device is usable by this process. */
int32_t b200_version(void);
int32_t b200_device_available(void);
/* Kernels this library has launched in this process so far (benchmarks report the difference
 * over their timed region; no reference counterpart). */
int64_t b200_launch_count(void);

/* ========================================================================================== */
/* HOST LAYER (no GPU needed)                                                                  */
/* ========================================================================================== */

/* ---- paged.BlockManager: src/kvcache/paged.zig:44-273 ------------------------------------ */
typedef struct b200_block_manager b200_block_manager;
b200_block_manager* b200_bm_create(uint64_t total_blocks);                       /* :53-84  init */
void b200_bm_destroy(b200_block_manager* bm);                                    /* :86-99  deinit */
int32_t b200_bm_can_allocate(const b200_block_manager* bm, uint64_t n);          /* :102-104 */
b200_status b200_bm_allocate_blocks(b200_block_manager* bm, uint64_t req_id, uint64_t n,
                                    uint64_t* out_ids);                          /* :108-137 */
void b200_bm_free_blocks(b200_block_manager* bm, uint64_t req_id);               /* :142-162 */
b200_status b200_bm_copy_on_write(b200_block_manager* bm, uint64_t block_id,
                                  uint64_t* out_id);                             /* :167-206 */
uint64_t b200_bm_free_count(const b200_block_manager* bm);                       /* :209-211 */
uint64_t b200_bm_used_count(const b200_block_manager* bm);                       /* :214-216 */
uint64_t b200_bm_total_blocks(const b200_block_manager* bm);
uint64_t b200_hash_block(uint64_t prev_hash, const uint32_t* token_ids, uint64_t n); /* :224-230 */
b200_status b200_bm_find_cached_prefix(b200_block_manager* bm, const uint32_t* token_ids,
                                       uint64_t n_tokens, uint64_t block_size, uint64_t* out_ids,
                                       uint64_t cap, uint64_t* out_n);           /* :234-265 */
b200_status b200_bm_register_block_hash(b200_block_manager* bm, uint64_t block_id,
                                        uint64_t hash);                          /* :268-272 */
/* Field access on block_pool.items[i] / req_to_blocks (the reference's tests write these). */
uint64_t b200_bm_get_ref(const b200_block_manager* bm, uint64_t block_id);       /* :34 ref_count */
void b200_bm_set_ref(b200_block_manager* bm, uint64_t block_id, uint64_t n);
int32_t b200_bm_is_used(const b200_block_manager* bm, uint64_t block_id);        /* :33 used */
uint64_t b200_bm_get_tokens_used(const b200_block_manager* bm, uint64_t block_id); /* :37 */
void b200_bm_set_tokens_used(b200_block_manager* bm, uint64_t block_id, uint64_t n);
void b200_bm_share(b200_block_manager* bm, uint64_t req_id, uint64_t block_id);  /* :48 req_to_blocks */
uint64_t b200_bm_blocks_of(const b200_block_manager* bm, uint64_t req_id, uint64_t* out_ids,
                           uint64_t cap);

/* ---- Request: src/scheduler.zig:101-187 --------------------------------------------------- */
enum { B200_REQ_WAITING = 0, B200_REQ_PREFILLING = 1, B200_REQ_DECODING = 2, B200_REQ_DONE = 3 };
typedef struct b200_request b200_request;
b200_request* b200_request_create(uint64_t id, const uint32_t* prompt, uint64_t n_prompt,
                                  uint64_t max_tokens, const uint32_t* stop_tokens,
                                  uint64_t n_stop);                              /* :123-142 init */
void b200_request_destroy(b200_request* r);                                      /* :144-147 */
uint64_t b200_request_id(const b200_request* r);
int32_t b200_request_state(const b200_request* r);                               /* :112 */
uint64_t b200_request_prefill_offset(const b200_request* r);                     /* :116 */
uint64_t b200_request_prompt_len(const b200_request* r);
uint64_t b200_request_seq_len(const b200_request* r);                            /* :165-167 */
int32_t b200_request_is_stop_token(const b200_request* r, uint32_t token);       /* :170-175 */
int32_t b200_request_has_pending_prefill(const b200_request* r);                 /* :178-180 */
uint64_t b200_request_current_prefill_chunk_len(const b200_request* r, uint64_t max_prefill_tokens); /* :183-186 */
uint64_t b200_request_generated(const b200_request* r, uint32_t* out, uint64_t cap); /* :111 */
uint64_t b200_request_block_ids(const b200_request* r, uint64_t* out, uint64_t cap); /* :113 */
uint64_t b200_request_prompt(const b200_request* r, uint32_t* out, uint64_t cap);     /* :110 */
/* The reference's tests construct mid-flight requests by writing the fields. */
void b200_request_force_state(b200_request* r, int32_t state, uint64_t prefill_offset,
                              const uint32_t* generated, uint64_t n_generated);
/* Sequence slot in a device KV pool bound to this request (-1 when none). */
int32_t b200_request_kv_slot(const b200_request* r);
/* Why a request ended before its stop condition: B200_OK, B200_ERR_CANCELLED, or the failure that was
 * its own (src/engine/engine_loop.zig:687-754 handleBatchError marks the request done and delivers the
 * error to its client). */
int32_t b200_request_error(const b200_request* r);

/* ---- scheduler-side BlockManager: src/scheduler.zig:22-95 --------------------------------- */
typedef struct b200_sched_bm b200_sched_bm;
typedef struct b200_kv b200_kv;
b200_sched_bm* b200_sched_bm_create(uint64_t total_blocks);                      /* :28-34 init */
b200_sched_bm* b200_sched_bm_create_with_real(b200_block_manager* real);         /* :37-43 initWithReal */
/* initWithReal against the device page pool: admission takes one page of the pool for a new
 * sequence slot, completion releases the sequence. */
b200_sched_bm* b200_sched_bm_create_with_kv(b200_kv* kv);
void b200_sched_bm_destroy(b200_sched_bm* bm);
/* Device-pool views only: take a sequence slot out of admission / give it back (releasing its pages);
 * sync re-reads the pool's free count after pages were allocated outside the scheduler. */
b200_status b200_sched_bm_park_slot(b200_sched_bm* bm, int32_t* out_slot);
b200_status b200_sched_bm_unpark_slot(b200_sched_bm* bm, int32_t slot);
b200_status b200_sched_bm_sync(b200_sched_bm* bm);
/* sync without a device read, for a caller that already holds the pool's free count (b200_llama_step
 * returns it after decode growth has taken pages). */
void b200_sched_bm_note_free(b200_sched_bm* bm, uint64_t free_pages);
int32_t b200_sched_bm_can_allocate(const b200_sched_bm* bm, uint64_t n);         /* :46-51 */
uint64_t b200_sched_bm_free_count(const b200_sched_bm* bm);                      /* :89-94 */
uint64_t b200_sched_bm_total_blocks(const b200_sched_bm* bm);
uint64_t b200_sched_bm_used_blocks(const b200_sched_bm* bm);

/* ---- Scheduler: src/scheduler.zig:222-387 -------------------------------------------------- */
typedef struct b200_scheduler b200_scheduler;
typedef struct b200_token_output { uint64_t request_id; uint32_t token; uint32_t _pad; } b200_token_output; /* :193-196 */
b200_scheduler* b200_scheduler_create(b200_sched_bm* bm, uint64_t max_prefill_tokens); /* :231-244 */
void b200_scheduler_destroy(b200_scheduler* s);                                  /* :246-249 */
b200_status b200_scheduler_add_request(b200_scheduler* s, b200_request* r);      /* :252-255 */
/* schedule(): fills caller arrays of capacity `cap` each (ScheduleResult, :202-216, :267-315). */
b200_status b200_scheduler_schedule(b200_scheduler* s, b200_request** prefill_out,
                                    uint64_t* n_prefill, b200_request** decode_out,
                                    uint64_t* n_decode, uint64_t cap, uint64_t* blocks_needed);
b200_status b200_scheduler_postprocess(b200_scheduler* s, const b200_token_output* outputs,
                                       uint64_t n);                              /* :328-381 */
/* A request leaves the scheduler before it has finished (cancellation, or a failure of its own): blocks
 * back to the pool, state done, `error` kept as the reason; the other requests are untouched
 * (src/engine/request_state.zig:182-189; src/engine/engine_loop.zig:687-754). */
b200_status b200_scheduler_remove(b200_scheduler* s, b200_request* r, int32_t error);
/* No reference counterpart (the reference admits on one free block, :242,291-293, and has no answer when
 * decode growth finds the pool empty): a running request returns all its blocks and goes back to the
 * head of the waiting queue; the tokens generated so far join its prompt, so its next prefill rebuilds
 * the same cache and its output continues where it stopped. */
b200_status b200_scheduler_preempt(b200_scheduler* s, b200_request* r);
/* While on, schedule() promotes no waiting request. */
void b200_scheduler_hold_admission(b200_scheduler* s, int32_t on);
/* Pages that one schedule() call may promise to newcomers (UINT64_MAX, the default, is the reference's
 * rule: one free block admits, :291-293).  With a budget a waiting request is promoted only while
 * ceil((prompt + 1) / 32) pages of it are left, in arrival order; the first request that does not fit
 * stops the promotions of that call. */
void b200_scheduler_set_admission_budget(b200_scheduler* s, uint64_t pages);
/* Running requests in admission order. */
uint64_t b200_scheduler_running(const b200_scheduler* s, b200_request** out, uint64_t cap);
uint64_t b200_scheduler_active_count(const b200_scheduler* s);                   /* :384-386 */
uint64_t b200_scheduler_waiting_count(const b200_scheduler* s);
uint64_t b200_scheduler_running_count(const b200_scheduler* s);

/* ---- batch_builder: src/batch_builder.zig:24-42, 47-83, 90-214, 253-256 ------------------- */
/* Host build of the flat batch (prefill requests first, then decode).  `chunked` = 0 reproduces
 * the reference (a prefilling request contributes all remaining prompt tokens, :50-66); 1 caps it
 * at its current chunk (src/scheduler.zig:183-186).  The T x T mask is not materialised: it is a
 * function of cu_seqlens (b200_is_attending); b200_batch_mask writes it out for parity checks. */
b200_status b200_batch_build(b200_request* const* prefill, uint64_t n_prefill,
                             b200_request* const* decode, uint64_t n_decode, int32_t chunked,
                             uint64_t max_prefill_tokens, uint32_t* tokens, int32_t* positions,
                             int32_t* row_to_req, uint64_t cap_tokens, int32_t* cu_seqlens,
                             uint64_t* total_tokens, uint64_t* num_requests);
int32_t b200_is_attending(const int32_t* cu_seqlens, uint64_t num_requests, uint64_t row,
                          uint64_t col);                                         /* :253-256 */
b200_status b200_batch_mask(const int32_t* cu_seqlens, uint64_t num_requests, float* mask,
                            uint64_t total_tokens);                              /* :138-177 */
/* Greedy sampler on a host logits row: first strict maximum (src/sampling.zig:22-39). */
uint32_t b200_greedy_host(const float* logits, uint64_t n);

/* ========================================================================================== */
/* DEVICE LAYER                                                                                */
/* ========================================================================================== */

/* ---- ragged batch packing on the GPU (replaces src/batch_builder.zig:122-205) ------------- */
/* One descriptor per request, in batch order. */
typedef struct b200_pack_desc {
  int32_t seq_slot;   /* sequence slot in the KV pool */
  int32_t count;      /* rows this request contributes (prefill chunk length, or 1) */
  int32_t base_pos;   /* position of its first row (src/batch_builder.zig:159-163) */
  int32_t src_offset; /* >= 0: offset into `prefill_tokens`; < 0: take last_token[seq_slot] */
} b200_pack_desc;
/* Exclusive prefix sum of counts -> cu_seqlens[R+1]; token_ids[T]; position_ids[T];
 * row_to_req[T]; row_seq[T] (slot per row); row_ctx[T] (= position + 1, the causal context of the
 * row); last_row[R] (row whose logits are sampled).  All pointers are device pointers. */
b200_status b200_pack_batch(const b200_pack_desc* d_desc, int32_t n_req,
                            const uint32_t* d_prefill_tokens, const uint32_t* d_last_token,
                            int32_t* d_cu_seqlens, uint32_t* d_token_ids, int32_t* d_position_ids,
                            int32_t* d_row_to_req, int32_t* d_row_seq, int32_t* d_row_ctx,
                            int32_t* d_last_row, int32_t total_rows, void* stream);

/* ---- Paged KV strategy on a device page pool ----------------------------------------------- */
/* Stands in for PagedKVCache (src/kvcache/paged.zig:305-1139) behind the KVCacheStrategy vtable
 * (src/kvcache/interface.zig:31-77), with the page allocator of paged.BlockManager (:44-206)
 * whose free stack, ref-counts and page tables live in device memory. */
enum { B200_KV_BF16 = 0, B200_KV_FP8_E4M3 = 1 };
typedef struct b200_kv_config {
  int32_t n_layers;
  int32_t n_kv_heads;        /* LayerConfig.num_kv_heads  src/kvcache/interface.zig:162-169 */
  int32_t head_dim;          /* LayerConfig.head_dim */
  int32_t page_size;         /* must be 32: src/kvcache/paged.zig:24 */
  int32_t n_pages;           /* pool size (BlockManager.total_blocks) */
  int32_t max_seqs;          /* sequence slots (LayerConfig.batch_size) */
  int32_t max_pages_per_seq; /* ceil(LayerConfig.max_seq_len / page_size) */
  int32_t kv_dtype;          /* B200_KV_BF16 | B200_KV_FP8_E4M3 (one f32 scale per page and kv head) */
  int32_t max_rows;          /* largest packed batch (rows) a step may carry */
  int32_t n_q_heads;         /* LayerConfig.num_heads (sizes the split-K scratch) */
  int32_t attn_scratch_chunks; /* split-K partial slots; 0 = n_pages/4 + max_rows + 8, which covers decode-only
                                * steps.  Steps with prefill chunks serve 16 / (q heads per kv head) rows per
                                * group and need, per group, ceil(context pages / 8) slots; a step that needs more
                                * slots than the pool holds is flagged B200_ERR_CAPACITY and changes nothing. */
} b200_kv_config;
b200_status b200_kv_create(const b200_kv_config* cfg, b200_kv** out);            /* :342-411 init, :1141-1186 factories */
void b200_kv_destroy(b200_kv* kv);                                               /* :1111-1138 deinit */
/* Pool size and number of sequence slots of a pool. */
b200_status b200_kv_dims(const b200_kv* kv, int32_t* n_pages, int32_t* max_seqs);
b200_status b200_kv_limits(const b200_kv* kv, int32_t* max_pages_per_seq, int32_t* page_size);
b200_status b200_kv_reset(b200_kv* kv);                                          /* :851-862 reset */
/* Install the order in which free pages will be popped (ids[0] first).  Default: 0,1,2,... */
b200_status b200_kv_set_free_order(b200_kv* kv, const int32_t* ids, int32_t n);
b200_status b200_kv_free_count(b200_kv* kv, int32_t* out);                       /* BlockManager.freeCount :209 */
/* allocateBlocks for one sequence slot (synchronous; used at admission). */
b200_status b200_kv_alloc(b200_kv* kv, int32_t seq, int32_t n, int32_t* out_ids); /* :108-137 */
/* freeBlocks for `n` sequence slots, in order. */
b200_status b200_kv_release(b200_kv* kv, const int32_t* seqs, int32_t n);        /* :142-162 */
/* Share the pages covering the first n_tokens of `src` with the empty slot `dst` (ref_count += 1,
 * the effect of findCachedPrefix :247-256). */
b200_status b200_kv_fork(b200_kv* kv, int32_t src, int32_t dst, int32_t n_tokens);
/* extend (VTable.extend, src/kvcache/interface.zig:60-69; src/kvcache/paged.zig:947-1109): sequence
 * src_seq of another pool of the same shape and element type becomes sequence dst_seq (an empty
 * slot) of this pool, with its own copies of the pages (reference count 1) in every layer.
 * Synchronous.  InsufficientBlocks when this pool cannot take the pages. */
b200_status b200_kv_extend(b200_kv* kv, int32_t dst_seq, b200_kv* src, int32_t src_seq);
b200_status b200_kv_rollback(b200_kv* kv, int32_t seq, int32_t to_len);          /* :864-877 */
/* filter: keep only the listed slots, release the rest (:879-945). */
b200_status b200_kv_filter(b200_kv* kv, const int32_t* keep, int32_t n_keep);
/* Step part 1 (device, asynchronous): grow page tables for a packed batch — per request, in
 * order: copy-on-write of a shared partially-filled last page (:167-206), then
 * ceil((len+count)/32) - held new pages (:525-531) — and build the page-touch work list for
 * append; the queued copy-on-write page copies (:186-200) are applied to every layer before it
 * returns control to the stream.  d_desc is the same array given to b200_pack_batch; a sequence
 * slot may appear at most once per step and n_req <= 4096. */
b200_status b200_kv_reserve(b200_kv* kv, const b200_pack_desc* d_desc, int32_t n_req, void* stream);
/* Step part 2: write K/V rows [T, n_kv_heads, head_dim] (bf16) of one layer into their pages
 * (:533-637).  K rows are expected already rotated, as updateAndFetch receives them. */
b200_status b200_kv_append(b200_kv* kv, int32_t layer, const void* d_k_rows, const void* d_v_rows,
                           int32_t total_rows, void* stream);
/* RoPE on q and k (in place, non-traditional, per-row positions, src/models/llama.zig:213-215) and the
 * append of the rotated K rows and the V rows in one launch: q [T, n_q_heads, head_dim], k and v
 * [T, n_kv_heads, head_dim] bf16, d_row_seq the sequence slot of every row (b200_pack_batch). */
b200_status b200_kv_rope_append(b200_kv* kv, int32_t layer, void* d_q, void* d_k_rows, const void* d_v_rows,
                                const int32_t* d_positions, const int32_t* d_row_seq, int32_t total_rows,
                                int32_t n_q_heads, float theta, void* stream);
/* The split-K partial sums of a matmul whose finish pass was left to the next kernel (b200_qmm_deferred):
 * f32 tiles [weight tile of 128 rows][token tile][split][tn tokens][128] in the library's matmul scratch, valid
 * until the next matmul on the stream.  pending = 0: nothing was deferred, y holds the result. */
typedef struct b200_qmm_partials {
  const float* d_ws;
  int32_t splits, tn, tts, nt, rows, n, pending;
} b200_qmm_partials;
/* b200_kv_rope_append fed from the partial sums of the fused q/k/v projection (no reference counterpart: the
 * seam between src/models/llama.zig:206-215 and the cache update, one launch less per layer): sums the K
 * splits in split order, rounds to bf16 exactly as the matmul's own finish pass would, rotates q and k, writes q
 * [T, n_q_heads, head_dim] into d_q (row stride q_stride elements) and the rotated k and v rows into their
 * pages.  Same bits as b200_qmm followed by b200_kv_rope_append.  bf16 pools with head_dim 128, and a
 * projection with n = (n_q_heads + 2 n_kv_heads) * 128 rows in q, k, v order; anything else returns
 * B200_ERR_UNSUPPORTED. */
b200_status b200_kv_rope_append_partials(b200_kv* kv, int32_t layer, const b200_qmm_partials* parts, void* d_q,
                                         int32_t q_stride, const int32_t* d_positions, const int32_t* d_row_seq,
                                         int32_t total_rows, int32_t n_q_heads, float theta, void* stream);
/* Introspection for bit-exact checks (synchronous). */
b200_status b200_kv_seq_len(b200_kv* kv, int32_t seq, int32_t* out_len);         /* :485-488 */
b200_status b200_kv_current_len(b200_kv* kv, int32_t* out_len);                  /* :842-849 currentLen */
b200_status b200_kv_block_table(b200_kv* kv, int32_t seq, int32_t* out_ids, int32_t cap,
                                int32_t* out_n_pages);
b200_status b200_kv_ref_counts(b200_kv* kv, int32_t* out, int32_t cap);
/* Reads and clears the device error word: 0, or a b200_status set by a kernel. */
b200_status b200_kv_error_word(b200_kv* kv, int32_t* out);
/* Tests only: the contiguous [len, n_kv_heads, head_dim] bf16 view updateAndFetch would return
 * (:705-802); FP8 pages are dequantised. */
b200_status b200_kv_gather(b200_kv* kv, int32_t layer, int32_t seq, void* d_k_out, void* d_v_out,
                           int32_t cap_rows, void* stream);
/* Raw E4M3 codes and scales of one page (FP8 pools; bit-exact checks). */
b200_status b200_kv_page_raw(b200_kv* kv, int32_t layer, int32_t page, void* h_k, void* h_v,
                             float* h_k_scales, float* h_v_scales);
/* Restoring pages saved elsewhere (PrefixDiskCache.loadBlock / restorePrefix,
 * src/kvcache/prefix_disk.zig:177-293): write one layer of a page from host memory (the inverse of
 * b200_kv_page_raw), and declare that the pages a slot holds (b200_kv_alloc) now carry n_tokens. */
b200_status b200_kv_page_load(b200_kv* kv, int32_t layer, int32_t page, const void* h_k,
                              const void* h_v, const float* h_k_scales, const float* h_v_scales);
b200_status b200_kv_set_len(b200_kv* kv, int32_t seq, int32_t n_tokens);

/* ---- split-K GQA paged-attention decode ----------------------------------------------------- */
/* Replaces gather + repeatHeads + softmax(QK^T/sqrt(D))V (src/kvcache/paged.zig:705-802,
 * src/models/llama.zig:231-270,303-323).  q, out: [T, n_q_heads, head_dim] bf16; row r attends to
 * the first d_row_ctx[r] cached tokens of slot d_row_seq[r]. */
b200_status b200_paged_attn_decode(b200_kv* kv, int32_t layer, const void* d_q,
                                   const int32_t* d_row_seq, const int32_t* d_row_ctx,
                                   int32_t total_rows, void* d_out, void* stream);
/* Same contract and results, for batches that hold prefill chunks (the block-diagonal causal mask
 * of src/batch_builder.zig:138-177 expressed as one context length per row, the chunk cursor of
 * src/scheduler.zig:183-186): consecutive rows of one sequence whose contexts grow by one token are
 * served together, so the cache is read once per group of rows instead of once per row. */
b200_status b200_paged_attn_prefill(b200_kv* kv, int32_t layer, const void* d_q,
                                    const int32_t* d_row_seq, const int32_t* d_row_ctx,
                                    int32_t total_rows, void* d_out, void* stream);

/* Tuning hook with no reference counterpart: pages per split-K chunk, 4..32; 0 (default) = 8, 16 or 32 chosen on
 * the device from the batch's mean context. */
void b200_set_attn_pages_per_chunk(int32_t n);
/* Tuning hook with no reference counterpart: b200_paged_attn_prefill serves batches of 1024 rows and more
 * with one chunk per group of rows and writes the normalised rows itself (default, 1); 0 keeps the chunked
 * path with f32 partials and a combine pass at every size (tests compare the two). */
void b200_set_attn_prefill_direct(int32_t on);
/* Tuning hook: 0 = automatic (tensor-core kernel for bf16 pools), 1 = force the CUDA-core kernel. */
void b200_set_attn_path(int32_t path);

/* ---- elementwise pieces of the layer (src/models/llama.zig) -------------------------------- */
b200_status b200_rmsnorm(const void* d_x, const void* d_weight, void* d_out, int32_t rows,
                         int32_t hidden, float eps, void* stream);                /* :462,473,592 */
/* In-place non-traditional RoPE on q [T,Hq,D] and k [T,Hkv,D] with per-row positions (:213-215). */
b200_status b200_rope(void* d_q, void* d_k, const int32_t* d_positions, int32_t rows,
                      int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim, int32_t q_stride,
                      int32_t k_stride, float theta, void* stream);
b200_status b200_embed_gather(const void* d_table, const uint32_t* d_ids, void* d_out, int32_t rows,
                              int32_t hidden, void* stream);                      /* :566 */
/* Greedy: first strict maximum per row of bf16 logits [rows, vocab] (src/sampling.zig:22-39). */
b200_status b200_argmax(const void* d_logits, int32_t rows, int32_t vocab, uint32_t* d_out,
                        void* stream);

/* ---- sampling beyond greedy (src/sampling.zig:42-242, 277-322) ------------------------------- */
/* One row of SamplerConfig (:277-285) plus the uniform variate in [0,1) that sampleFromProbs (:258-268)
 * draws: the caller draws it from its own per-request PRNG, so the token is a pure function of the
 * row.  temperature <= 0 is greedy (:313-314); top_p >= 1 with top_k >= vocab samples the full
 * softmax in index order (temperatureSample, :42-72); everything else is topKTopPSampler (:175-242):
 * scores = logit / temperature sorted descending (equal scores keep index order), softmax over the
 * top k, cut after the first prefix whose cumulative probability exceeds top_p, renormalise, sample.
 * top_k <= 0 means no limit (the reference indexes an empty slice there). */
typedef struct b200_sample_params {
  float temperature;
  float top_p;
  float repetition_penalty; /* applied when > 1 and the row has context tokens (:301-309, 328-354) */
  float uniform;
  int32_t top_k;
  int32_t _pad;
} b200_sample_params;
/* d_logits [rows, vocab], bf16 (logits_f32 = 0) or f32 (1), widened to f32 like the reference's
 * astype (src/generation.zig:124-141).  d_ctx_tokens / d_ctx_offsets[rows+1] (optional) give each row's
 * token history for the repetition penalty, applied once per occurrence; d_scratch [rows, vocab] f32
 * is required with them.  d_logprobs (optional) receives log softmax of the (penalised, unscaled)
 * logits at the sampled token (computeLogprob, :355-375).  Sums over the whole vocabulary are
 * parallel reductions; sums over the sorted top-k prefix run in the reference's order. */
b200_status b200_sample_rows(const void* d_logits, int32_t logits_f32, int32_t rows, int32_t vocab,
                             const b200_sample_params* d_params, const uint32_t* d_ctx_tokens,
                             const int32_t* d_ctx_offsets, float* d_scratch, uint32_t* d_tokens,
                             float* d_logprobs, void* stream);
/* std.Random.DefaultPrng as SamplerConfig.init seeds it (:287-296): xoshiro256++ whose state comes
 * from SplitMix64(seed), and Random.float(f32) (23 mantissa bits, exponent from the leading-zero
 * count of the remaining bits).  Both belong to the Zig standard library, not to the reference. */
void b200_prng_seed(uint64_t seed, uint64_t state[4]);
uint64_t b200_prng_next_u64(uint64_t state[4]);
float b200_prng_next_f32(uint64_t state[4]);

/* ---- dequant-fused quantised matmul --------------------------------------------------------- */
/* y[T,N] = x[T,K] . dequant(W[N,K])^T  (quantizedMatmul call sites src/models/llama.zig:127,367,596;
 * gatherQmm src/models/deepseek_v4.zig:976).  Weights are repacked once into a tile-major device
 * layout; the handle owns that memory. */
enum { B200_Q_AFFINE4_G64 = 0, B200_Q_MXFP4_G32 = 1, B200_Q_BF16 = 2 };
typedef struct b200_qweight b200_qweight;
/* affine: packed uint32 [N, K/8] (8 nibbles per word, least significant first), scales and biases
 * bf16 [N, K/64]  (src/kvcache/paged.zig:358,1199-1208; src/models/llama_loader.zig:262-279).
 * mxfp4: packed uint8 [N, K/2] (low nibble = even element), E8M0 scales uint8 [N, K/32], no
 * biases (src/models/deepseek_v4_loader.zig:121-122,839-920).  Host pointers.
 * bf16  : dense bf16 [N, K] in h_packed, no scales (the unquantised branch of `linear`,
 *         src/models/llama.zig:129).
 * n_experts > 1 stacks [E, N, K] for grouped use. */
b200_status b200_qweight_create(int32_t mode, int32_t n_experts, int32_t n, int32_t k,
                                const void* h_packed, const void* h_scales, const void* h_biases,
                                b200_qweight** out);
/* Synthetic weights generated on the device (benchmarks with random-init models): uniform random
 * codes with fixed plausible scales.  N a multiple of 128, K of 64. */
b200_status b200_qweight_random(int32_t mode, int32_t n_experts, int32_t n, int32_t k, uint32_t seed,
                                b200_qweight** out);
/* The inverse of b200_qweight_create for one expert of a handle: host buffers in the layouts
 * b200_qweight_create takes (checks of weights that were generated on the device). */
b200_status b200_qweight_export(const b200_qweight* w, int32_t expert, void* h_packed, void* h_scales,
                                void* h_biases);
void b200_qweight_destroy(b200_qweight* w);
enum { B200_EPI_NONE = 0, B200_EPI_RESIDUAL = 1, B200_EPI_SWIGLU = 2 };
enum { B200_QMM_AUTO = 0, B200_QMM_SIMT = 1, B200_QMM_TCGEN05 = 2, B200_QMM_MMA = 3, B200_QMM_TCGEN05_X2 = 4,
       B200_QMM_TCGEN05_TMEM_A = 5, B200_QMM_MXFP4_BLOCK_SCALED = 6, B200_QMM_MMA_I8 = 7 };
/* Tuning hook (no reference counterpart): 1 sends the grouped (MoE) matmuls through the kernel that
 * keeps dequantised weights in tensor memory. */
void b200_set_qmm_grouped_tmem_a(int32_t on);
/* 1 sends the grouped matmuls of MXFP4 weights (K a multiple of 128, work items of up to 128 rows)
 * through tcgen05.mma kind::mxf8f6f4 with block scaling: the E2M1 codes and E8M0 scales go to the
 * tensor cores as they are, the bf16 activations as two E4M3 halves.  The same kernel serves b200_qmm
 * with path B200_QMM_MXFP4_BLOCK_SCALED.  The weight handle builds a second copy of itself (plain
 * row-major codes + scale atoms) on first use. */
void b200_set_qmm_grouped_block_scaled(int32_t on);
/* Tuning hook: 1 (default) runs the block-scaled MXFP4 path as persistent CTAs walking a list of work items
 * (tile pair x token tile or expert item x K range), 0 as one CTA per work item. */
void b200_set_qmm_mx_persistent(int32_t on);
/* epilogue NONE: y = xW^T.  RESIDUAL: y = residual + xW^T.  SWIGLU: W holds gate and up rows
 * interleaved (row 2i = gate_i, 2i+1 = up_i); y[T, N/2] = silu(min(g,L)) * clip(u,+-L) with
 * L = swiglu_limit (0 = unclipped)  (src/models/llama.zig:396-415; deepseek_v4.zig:947-966). */
b200_status b200_qmm(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y,
                     int32_t epilogue, const void* d_residual, float swiglu_limit, int32_t path,
                     void* stream);

/* b200_qmm with epilogue NONE whose split-K finish pass may be left to the caller's next kernel (no reference
 * counterpart).  defer = 0: exactly b200_qmm.  defer != 0: when the chosen kernel splits K, the finish pass is not
 * launched, out->pending = 1 and out describes the partial sums (d_y is NOT written); when it does not split K,
 * d_y is written and out->pending = 0. */
b200_status b200_qmm_deferred(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y, int32_t defer,
                              void* stream, b200_qmm_partials* out);

/* y = residual + x W^T and normed = rmsnorm(y) * norm_weight in one call: the pair that closes the
 * attention and the FFN half of a block (src/models/llama.zig:466-477: residual add, then the next
 * RMSNorm).  When the matmul splits K its finish pass writes both; otherwise the row kernel follows.
 * d_y may alias d_residual. */
b200_status b200_qmm_residual_norm(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y,
                                   const void* d_residual, const void* d_norm_weight, float eps,
                                   void* d_normed, void* stream);

/* Reads and clears the matmul kernels' error words (set when a bounded wait ran out): the word of
 * b200_qmm and the grouped launches, and the word of b200_qmm_static_scratch on the current device. */
b200_status b200_qmm_error_word(int32_t* out);
/* Test hook: writes `value` into the error word of b200_qmm (static_scratch_word = 0) or of
 * b200_qmm_static_scratch (1), so that the read-and-clear path can be checked without a kernel that
 * times out. */
b200_status b200_qmm_debug_set_error_word(int32_t value, int32_t static_scratch_word);
/* Test hook: launches a kernel whose one bounded wait (at most `polls` polls, 1..2^20) is on a barrier
 * that nothing completes.  The wait runs out, the kernel sets the matmul error word the way the matmul
 * kernels do and returns normally; b200_qmm_error_word then reports B200_ERR_DEVICE_FLAGGED and the
 * library stays usable. */
b200_status b200_qmm_debug_wait_runs_out(int32_t polls, void* stream);
/* No counterpart in the reference.  The tensor-core matmul of b200_qmm for hosts that must not
 * allocate after start-up (all HBM already given to the KV pool, a step being captured into a CUDA
 * graph or running beside other streams, where cudaMalloc would fail or stall the device): its
 * split-K scratch is a fixed 32 MiB array inside the library instead of a buffer grown on demand,
 * and the call allocates nothing.  Problems whose scratch (K-splits x round_up(rows, token tile) x
 * round_up(N,128) x 4 bytes, the token tile being min(256, round_up(rows,16)) rows, so 257 rows count
 * as 512) exceeds the array are refused with B200_ERR_CAPACITY.  The first call on a device resolves
 * the array's address and opts the kernel into large shared memory there, and should come before any
 * stream capture; all calls share the array, so calls that overlap on the GPU race.  A bounded wait
 * that runs out inside its kernels is reported through b200_qmm_error_word. */
b200_status b200_qmm_static_scratch(const b200_qweight* w, const void* d_x, int32_t rows, void* d_y,
                                    int32_t epilogue, const void* d_residual, float swiglu_limit,
                                    void* stream);

/* ---- LLaMA-architecture decode step over a packed ragged batch --------------------------------- */
/* Stands in for ModelVTable.forward + the greedy branch of generateBatchStep
 * (src/generation.zig:47-53,104-145) with LlamaModel.forward underneath
 * (src/models/llama.zig:556-609). */
typedef struct b200_llama_config {
  int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab; /* LlamaConfig, src/models/llama.zig:40-70 */
  int32_t max_rows;  /* largest packed batch (rows) */
  int32_t max_reqs;  /* most requests in one step */
  int32_t max_seqs;  /* sequence slots of the page pool it will run on */
  float rms_eps;
  float rope_theta;
} b200_llama_config;
typedef struct b200_llama b200_llama;
enum { B200_W_Q = 0, B200_W_K = 1, B200_W_V = 2, B200_W_O = 3, B200_W_GATE = 4, B200_W_UP = 5, B200_W_DOWN = 6,
       B200_W_LM_HEAD = 7 };
b200_status b200_llama_create(const b200_llama_config* cfg, b200_llama** out);
void b200_llama_destroy(b200_llama* m);
/* One projection matrix in the reference's layout ([out, in]; quantised triples as produced by the
 * loader, src/models/llama_loader.zig:245-279).  q/k/v and gate/up are fused at finalize. */
b200_status b200_llama_set_linear(b200_llama* m, int32_t layer, int32_t which, int32_t mode,
                                  const void* h_packed, const void* h_scales, const void* h_biases);
b200_status b200_llama_set_embedding(b200_llama* m, const void* h_bf16);          /* [vocab, hidden] */
/* layer < 0: final norm; which: 0 = attention norm, 1 = ffn norm.  bf16 [hidden]. */
b200_status b200_llama_set_norm(b200_llama* m, int32_t layer, int32_t which, const void* h_bf16);
b200_status b200_llama_finalize(b200_llama* m);
/* Synthetic random-init model generated on the device (benchmarks). */
b200_status b200_llama_random_init(b200_llama* m, int32_t mode, uint32_t seed);
/* One engine step with host buffers: descriptors and prefill tokens in, one greedy token per
 * request out (first strict max, src/sampling.zig:22-39).  Copies, runs the whole stack, copies
 * back and synchronises the stream.  out_free_pages (optional) receives the pool's free count. */
b200_status b200_llama_step(b200_llama* m, b200_kv* kv, const b200_pack_desc* h_desc, int32_t n_req,
                            const uint32_t* h_prefill_tokens, int32_t n_prefill_tokens,
                            uint32_t* h_next_tokens, int32_t* out_free_pages, void* stream);
/* The same step on device-resident inputs, asynchronous on `stream` (no copies, no sync). */
b200_status b200_llama_forward(b200_llama* m, b200_kv* kv, const b200_pack_desc* d_desc, int32_t n_req,
                               int32_t total_rows, const uint32_t* d_prefill_tokens, void* stream);
void b200_llama_device_buffers(b200_llama* m, b200_pack_desc** d_desc, uint32_t** d_prefill,
                               uint32_t** d_next);
/* Sampler rows for the requests of the NEXT b200_llama_step, in descriptor order (one use): that
 * step draws its tokens with b200_sample_rows instead of the argmax.  Rows with temperature <= 0
 * stay greedy.  b200_llama_last_logprobs returns the log-probabilities of that step's tokens. */
b200_status b200_llama_set_samplers(b200_llama* m, const b200_sample_params* h_rows, int32_t n_req);
b200_status b200_llama_last_logprobs(b200_llama* m, float* h_out, int32_t n_req);
/* bf16 logits [n_req, vocab] of the last step's sampled rows (tests). */
b200_status b200_llama_last_logits(b200_llama* m, void* h_bf16_out, int32_t n_req);
int64_t b200_llama_launch_count(const b200_llama* m);
/* Decode-only steps are replayed as CUDA graphs by default (on = 0 turns that off). */
void b200_llama_enable_graphs(b200_llama* m, int32_t on);
/* The step feeds RoPE + KV append from the q/k/v projection's split-K partial sums where it can
 * (b200_kv_rope_append_partials; default on).  0 keeps the projection's own finish pass and b200_kv_rope_append
 * (tests compare the two: same tokens, same pages). */
void b200_llama_set_fused_qkv_rope(b200_llama* m, int32_t on);
/* CUDA-event timing of the step's kernels by category (0 attention, 1 matmuls, 2 rope + KV append,
 * 3 the rest); collect() synchronises, fills ms[4] and calls[4], and clears the record.  Stands in
 * for the reference's per-step timing logs (src/models/expert_stream.zig:36-51 TokenStepMetrics). */
void b200_llama_profile_enable(b200_llama* m, int32_t on);
b200_status b200_llama_profile_collect(b200_llama* m, double* ms, int64_t* calls);

/* ---- engine step: schedule -> pack -> model step -> postprocess ------------------------------- */
/* The Engine_Step loop of src/scheduler.zig:7-10 wired to a forward pass (the reference leaves
 * it unwired, docs/en/technical/continuous-batching-design.md:187; its production loop is
 * src/engine/engine_loop.zig:225-281,532-682).  The scheduler's BlockManager is the device pool.
 * Prefill is chunked by max_prefill_tokens (src/scheduler.zig:183-186). */
typedef struct b200_engine b200_engine;
b200_engine* b200_engine_create(b200_llama* model, b200_kv* kv, uint64_t max_prefill_tokens);
void b200_engine_destroy(b200_engine* e);
b200_status b200_engine_submit(b200_engine* e, uint64_t id, const uint32_t* prompt, uint64_t n_prompt,
                               uint64_t max_tokens, const uint32_t* stop_tokens, uint64_t n_stop);
/* One step; `out` receives the tokens that joined a request's output this step (checked to fit `cap`
 * before anything is written to the cache).  Page-table growth is budgeted on the host against the
 * pool's free count before the model step: decode rows first, then prefill chunks; a request whose
 * growth does not fit is left out of the step and keeps its cursor; when nothing fits, the youngest
 * running request is preempted (b200_scheduler_preempt) — or fails on its own if it is alone.  A step
 * that a kernel flags all the same changes neither the pool nor any sequence's next input token, so
 * the caller may step again. */
b200_status b200_engine_step(b200_engine* e, b200_token_output* out, uint64_t cap, uint64_t* n_out,
                             void* stream);
uint64_t b200_engine_active_count(const b200_engine* e);
b200_status b200_engine_result(const b200_engine* e, uint64_t id, uint32_t* out, uint64_t cap,
                               uint64_t* n, int32_t* done);
void b200_engine_forget(b200_engine* e, uint64_t id);
/* Cancels a request wherever it is (waiting, mid-prefill, decoding): it leaves the scheduler at once,
 * its pages return to the pool, the tokens it has produced stay readable and its status becomes
 * B200_ERR_CANCELLED (RequestState.cancelled, src/engine/request_state.zig:118,182-189, checked by the
 * engine thread at src/engine/engine_loop.zig:240-243).  Called between steps. */
b200_status b200_engine_cancel(b200_engine* e, uint64_t id);
/* B200_OK, or why the request ended early: B200_ERR_CANCELLED, B200_ERR_CAPACITY (its sequence reached
 * the length a page table holds) or B200_ERR_INSUFFICIENT_BLOCKS (it does not fit the pool even alone).
 * A request that fails this way leaves the batch on its own; the others go on
 * (src/engine/engine_loop.zig:687-754). */
b200_status b200_engine_request_status(const b200_engine* e, uint64_t id, int32_t* status);
/* Page-pool pressure so far: request-steps left out because their page growth did not fit, running
 * requests sent back to the waiting queue to free pages (their cache is recomputed when they are
 * admitted again), requests that failed on their own.  While running requests are short of pages no
 * new request is admitted. */
void b200_engine_pressure_stats(const b200_engine* e, uint64_t* deferred, uint64_t* preempted, uint64_t* failed);
int32_t b200_engine_free_pages(const b200_engine* e);
/* Request ids of the last step's batch in descriptor order (prefill chunks first, then decode rows,
 * src/batch_builder.zig:100-111): row i of b200_llama_last_logits belongs to ids[i].  Returns the
 * batch size. */
uint64_t b200_engine_last_batch(const b200_engine* e, uint64_t* ids, uint64_t cap);
/* Prefix pages that outlive requests (RestoredPrefix, src/kvcache/prefix_disk.zig:15-29, 246-293): the
 * caller parks a sequence slot, fills it (b200_kv_alloc + b200_kv_page_load + b200_kv_set_len, e.g.
 * from blocks restored from disk) and publishes it with the token ids its pages hold; with prefix
 * sharing on, later requests take over its full blocks by reference count exactly as they do from a
 * live request.  drop releases the slot and its pages (pages still shared stay alive through their
 * reference counts).  b200_engine_request_slot gives the slot of a running request (-1 if none), so
 * that its prompt blocks can be saved before it finishes. */
b200_status b200_engine_park_slot(b200_engine* e, int32_t* out_slot);
b200_status b200_engine_publish_prefix(b200_engine* e, int32_t slot, const uint32_t* token_ids,
                                       uint64_t n_tokens);
b200_status b200_engine_drop_prefix(b200_engine* e, int32_t slot);
int32_t b200_engine_request_slot(const b200_engine* e, uint64_t id);
/* Sampler of one request (SamplerConfig, src/sampling.zig:277-296): temperature, top-k, top-p and a
 * PRNG seeded like SamplerConfig.init.  A request without one is greedy.  One uniform variate is
 * drawn per token that joins the request's output, so a request's variates do not depend on what
 * it is batched with.  No repetition penalty on this path. */
b200_status b200_engine_set_sampler(b200_engine* e, uint64_t id, float temperature, int32_t top_k,
                                    float top_p, uint64_t seed);
/* Prefix sharing (off by default): a request about to start its prefill takes over, by reference
 * count, the full 32-token prompt blocks that a live request with the same chained block hashes has
 * already prefilled (findCachedPrefix, src/kvcache/paged.zig:234-265); its own appends copy a shared
 * page on write (:167-206).  shared_tokens reports how many prompt tokens a request took over. */
void b200_engine_set_prefix_sharing(b200_engine* e, int32_t on);
/* Cap on the tokens of one step (0 = none, as in the reference scheduler, which sends a chunk of every
 * prefilling request): prefill chunks beyond the budget wait for a later step; decode rows always run. */
void b200_engine_set_max_step_tokens(b200_engine* e, uint64_t n);
uint64_t b200_engine_shared_tokens(const b200_engine* e, uint64_t id);

/* ---- mixture of experts ------------------------------------------------------------------------ */
/* Top-k routing (MoERouter.topkRoute, src/moe_router.zig:55-103; DSV4Gate.forward scoring, bias and
 * weights, src/models/deepseek_v4.zig:555-681).  logits [N,E] bf16 (or f32); scoring 0 = softmax,
 * 1 = sigmoid, 2 = sqrt(softplus); bias (optional, f32 [E]) steers the choice only; weights come
 * from the unbiased scores, renormalised over the selection unless softmax, times route_scale.
 * Output per token in ascending (score, expert index) order — the last k of an ascending stable
 * argsort.  counts (optional, i32 [E]) receives the per-expert histogram. */
b200_status b200_moe_route(const void* d_logits, int32_t logits_are_f32, const float* d_bias,
                           int32_t n_tokens, int32_t n_experts, int32_t k, int32_t scoring,
                           float route_scale, uint32_t* d_indices, float* d_weights,
                           int32_t* d_counts, void* stream);
/* Stable grouping of the N*k assignments by expert (argsort(flat indices), argsort(order),
 * src/models/deepseek_v4.zig:747-784): offsets [E+1], order [N*k], inv_order [N*k], plus the work
 * items ({expert, first row, rows, 0} as 4 x i32; capacity E + ceil(N*k / tile_rows)) that the
 * grouped matmul consumes. */
b200_status b200_moe_group(const uint32_t* d_indices, const int32_t* d_counts, int32_t n_tokens,
                           int32_t k, int32_t n_experts, int32_t tile_rows, int32_t* d_offsets,
                           int32_t* d_order, int32_t* d_inv_order, void* d_items,
                           int32_t* d_n_items, void* stream);
/* x_sorted[p] = x[order[p] / k]; row_scales[p] = weights[order[p]]  (expandTokens + the gathers of
 * src/moe_router.zig:111-132, deepseek_v4.zig:760-784). */
b200_status b200_moe_gather(const void* d_x, const int32_t* d_order, const float* d_weights,
                            int32_t n_assign, int32_t k, int32_t hidden, void* d_x_sorted,
                            float* d_row_scales, void* stream);
/* dst[r] = src[idx[r]] for bf16 rows (regrouping rows received from other ranks into expert-major
 * order in the expert-parallel layout; no reference counterpart — the reference has no expert
 * parallelism, src/models/expert_stream.zig streams experts from SSD instead). */
b200_status b200_moe_gather_rows(const void* d_src, const int32_t* d_idx, void* d_dst, int32_t rows,
                                 int32_t hidden, void* stream);
/* Ragged grouped quantised matmul over the expert-sorted rows (gather_qmm with sorted indices,
 * src/models/deepseek_v4.zig:787-805,968-979); w stacks n_experts matrices; row_scales (optional)
 * multiplies each output row in the epilogue. */
b200_status b200_moe_grouped_qmm(const b200_qweight* w, const void* d_x_sorted, int32_t rows,
                                 void* d_y_sorted, int32_t epilogue, const float* d_row_scales,
                                 float swiglu_limit, const void* d_items, const int32_t* d_n_items,
                                 int32_t max_items, int32_t tile_rows, void* stream);
/* out[t] = sum_j y_sorted[inv_order[t*k + j]] (+ shared_out[t])  (reduceExperts,
 * src/moe_router.zig:139-164; deepseek_v4.zig:809-819,1051). */
b200_status b200_moe_combine(const void* d_y_sorted, const int32_t* d_inv_order, int32_t n_tokens,
                             int32_t k, int32_t hidden, const void* d_shared_out, void* d_out,
                             void* stream);
/* One MoE layer = DSV4MoE.forward (src/models/deepseek_v4.zig:1010-1056).  Weight handles are
 * borrowed: gate dense bf16 [E, hidden]; experts_gate_up stacks E x [2*inter, hidden] with gate
 * and up rows interleaved; experts_down E x [hidden, inter]; shared_* optional. */
typedef struct b200_moe_config {
  int32_t hidden, n_experts, inter, top_k;
  int32_t scoring;       /* 0 softmax, 1 sigmoid, 2 sqrt-softplus */
  int32_t tile_rows;     /* token tile of the grouped matmul: multiple of 16, 16..256; up to 112 the block-scaled
                          * MXFP4 kernel keeps two accumulator sets and overlaps an item's epilogue with the
                          * next item's MMAs (112 measured best for experts of about a hundred rows) */
  int32_t max_tokens;
  float route_scale;
  float swiglu_limit;        /* routed experts: 10 in the reference (deepseek_v4.zig:64) */
  float shared_swiglu_limit; /* shared expert (0 = unclipped) */
  /* Expert parallelism (ep_world = 0: off, every expert is local; a group of one rank is allowed and runs
   * the same code path).  n_experts stays the number of routed
   * experts of the model; the expert weight handles then stack the n_experts / ep_world experts of this
   * rank (global expert e lives on rank e / (n_experts / ep_world)), max_tokens is the most tokens ONE
   * rank brings to a step, and the layer runs through b200_moe_forward_ep. */
  int32_t ep_rank, ep_world;
} b200_moe_config;
typedef struct b200_moe b200_moe;
b200_status b200_moe_create(const b200_moe_config* cfg, const b200_qweight* gate, const float* h_bias,
                            const b200_qweight* experts_gate_up, const b200_qweight* experts_down,
                            const b200_qweight* shared_gate_up, const b200_qweight* shared_down,
                            b200_moe** out);
void b200_moe_destroy(b200_moe* m);
b200_status b200_moe_forward(b200_moe* m, const void* d_x, int32_t n_tokens, void* d_out, void* stream);
b200_status b200_moe_last_routing(b200_moe* m, int32_t n_tokens, uint32_t* h_indices, float* h_weights,
                                  int32_t* h_offsets);


/* ---- expert parallelism ---------------------------------------------------------------------------- */
/* No reference counterpart: the reference keeps all experts on one device and streams them from SSD
 * (src/models/expert_stream.zig:400-613).  The routed experts are sharded over `world` ranks, one
 * process per GPU; DSV4SwitchGLU is cut at its two argsorts (src/models/deepseek_v4.zig:747-784 sort by
 * expert -> dispatch; :809-819 unsort and sum over k -> combine).  The communicator is NCCL, loaded at
 * run time; rank 0 makes the 128-byte id and the host hands it to every rank by its own means. */
enum { B200_EP_UNIQUE_ID_BYTES = 128 };
typedef struct b200_ep b200_ep;
b200_status b200_ep_unique_id(uint8_t* out_128_bytes);                   /* ncclGetUniqueId */
b200_status b200_ep_create(int32_t rank, int32_t world, const uint8_t* unique_id, b200_ep** out); /* collective */
void b200_ep_destroy(b200_ep* ep);
int32_t b200_ep_rank(const b200_ep* ep);
int32_t b200_ep_world(const b200_ep* ep);
int32_t b200_ep_nccl_version(void);
/* dispatch: every rank's n_rows token rows [n_rows, hidden] bf16 -> all ranks' rows, rank-major
 * [world * n_rows, hidden] (an all-gather: with top-6 routing over 8 ranks nearly every rank needs
 * nearly every token, and no per-destination count has to reach the host first).  Queued on `stream`. */
b200_status b200_ep_dispatch(b200_ep* ep, const void* d_rows, void* d_rows_all, int32_t n_rows, int32_t hidden,
                             void* stream);
/* plan: the grouping of deepseek_v4.zig:747-784 restricted to this rank's experts.  d_indices [N, k] and
 * d_counts [n_experts] come from b200_moe_route over the tokens of all ranks; outputs: offsets
 * [E_local + 1], order (row p of the grouped matmul is assignment order[p]; offsets[E_local] rows exist),
 * inv_order [N * k] (-1 where another rank serves the assignment), work items, d_local_idx [N * k] scratch. */
b200_status b200_ep_plan(const uint32_t* d_indices, const int32_t* d_counts, int32_t n_tokens, int32_t k,
                         int32_t n_experts, int32_t rank, int32_t world, int32_t tile_rows, uint32_t* d_local_idx,
                         int32_t* d_offsets, int32_t* d_order, int32_t* d_inv_order, void* d_items,
                         int32_t* d_n_items, void* stream);
/* combine: d_partial_all [world * n_rows, hidden] f32 holds, for the tokens of all ranks, the sum of the
 * outputs of THIS rank's experts; the reduce-scatter leaves in d_sum [n_rows, hidden] f32 the complete
 * sums over k of this rank's own tokens (reduceExperts, src/moe_router.zig:139-164).  Queued on `stream`. */
b200_status b200_ep_combine(b200_ep* ep, const float* d_partial_all, float* d_sum, int32_t n_rows, int32_t hidden,
                            void* stream);
/* DSV4MoE.forward (src/models/deepseek_v4.zig:1010-1056) for a layer created with ep_world > 1: dispatch,
 * replicated routing, plan, grouped matmuls on the local experts, combine, shared expert.  Every rank
 * calls it with the same n_tokens.  Two collectives, no host synchronisation. */
b200_status b200_moe_forward_ep(b200_moe* m, b200_ep* ep, const void* d_x, int32_t n_tokens, void* d_out,
                                void* stream);
/* Host-side watchdog: waits until the work queued on `stream` so far has finished, at most timeout_ms
 * (negative = no limit), polling ncclCommGetAsyncError; on an error or when the time is up the
 * communicator is aborted (ncclCommAbort), the GPU comes back to the caller and B200_ERR_DEVICE_FLAGGED is
 * returned.  After an abort the handle only accepts b200_ep_destroy. */
b200_status b200_ep_wait(b200_ep* ep, void* stream, int32_t timeout_ms);
b200_status b200_ep_abort(b200_ep* ep);
/* The watchdog's loop on its own, over caller-supplied operations (each gets ctx): done() != 0 when the
 * work has finished, async_error() != 0 when the communicator reports an error, abort() tears it down. */
typedef struct b200_ep_watch_ops {
  int (*done)(void* ctx);
  int (*async_error)(void* ctx);
  void (*abort)(void* ctx);
  void* ctx;
} b200_ep_watch_ops;
enum { B200_EP_WATCH_DONE = 0, B200_EP_WATCH_ERROR = 1, B200_EP_WATCH_TIMEOUT = 2 };
int32_t b200_ep_watch(const b200_ep_watch_ops* ops, int32_t timeout_ms, int32_t poll_us);

#ifdef __cplusplus
}
#endif
#endif /* DMLX_B200_H */
