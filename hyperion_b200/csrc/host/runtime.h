/* C interface of the host runtime: cache bookkeeping, scheduler and step assembly.
 *
 * Every function returns 0 on success or one of the codes below; hb_host_last_error() then gives the
 * text (per thread). Requests are named by 64-bit keys that the caller chooses. Nothing here touches
 * a device: the step assembler writes 32-bit words into a host buffer the caller owns (pinned memory
 * in the engine) and the caller copies it.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB_HOST_OK 0
#define HB_HOST_OUT_OF_PAGES 1
#define HB_HOST_CACHE_ERROR 2
#define HB_HOST_BAD_ARGUMENT 3
#define HB_HOST_BAD_STEP 4
#define HB_HOST_QUEUE_FULL 5
#define HB_HOST_SCHEDULER_ERROR 6
#define HB_HOST_BAD_FILE 7

const char* hb_host_last_error(void);

/* ---- a pool of pages on its own ---- */
typedef struct HbPool HbPool;
int hb_pool_new(int num_pages, HbPool** out);
void hb_pool_delete(HbPool* pool);
int hb_pool_available(const HbPool* pool);
int hb_pool_take(HbPool* pool, int* page);
int hb_pool_give_back(HbPool* pool, int page);
int hb_pool_is_held(const HbPool* pool, int page);
int hb_pool_check(const HbPool* pool);

/* ---- cache index ---- */
typedef struct HbCache HbCache;
int hb_cache_new(int page_size, int num_pages, int max_requests, int n_groups, const int* windows, HbCache** out);
void hb_cache_delete(HbCache* cache);
int hb_cache_has(const HbCache* cache, int64_t key);
int hb_cache_add(HbCache* cache, int64_t key, int* slot);
int hb_cache_length(const HbCache* cache, int64_t key, int* length);
int hb_cache_slot(const HbCache* cache, int64_t key, int* slot);
int hb_cache_table_size(const HbCache* cache, int group, int64_t key, int* size);
int hb_cache_table(const HbCache* cache, int group, int64_t key, int* pages, int capacity);
int hb_cache_pages_needed(const HbCache* cache, int64_t key, int new_tokens, int* per_group);
int hb_cache_extend_all(HbCache* cache, int n, const int64_t* keys, const int* counts);
/* released: (group, page) pairs, at most capacity of them are written; n_released counts all */
int hb_cache_advance(HbCache* cache, int64_t key, int new_tokens, int* released, int capacity, int* n_released);
int hb_cache_advance_all(HbCache* cache, int n, const int64_t* keys, const int* counts);
int hb_cache_free(HbCache* cache, int64_t key);
int hb_cache_free_pages(const HbCache* cache, int group, int* pages);
int hb_cache_live(const HbCache* cache, int64_t* keys, int capacity, int* n_live);
int hb_cache_lengths(const HbCache* cache, int n, const int64_t* keys, int* lengths, int* slots); /* -1 for unknown keys */
int hb_cache_check(const HbCache* cache);
/* The most pages of one group a request of `tokens` tokens can hold when no step brings it more than largest_portion tokens. */
int hb_cache_worst_case_pages(int page_size, int window, int tokens, int largest_portion, int* pages);

/* ---- step assembly ----
 * Writes the arrays every step carries, each starting at a multiple of 4 words, into out[*cursor ...]:
 *   0 token_ids [T]   1 positions [T]   2 token_row [T]   3 row_start [R + 1]   4 slots [R]   5 want [W]
 *   6 + g: block table of group g [R, width_g], missing pages as -1
 * width_g is the longest table of the step's rows, at least 1, rounded up to a multiple of table_step when
 * that is positive, and to -table_step times a power of two when it is negative. layout receives (offset, count, rows, columns) per array; *cursor moves past them.
 * Positions start at each request's current length; call it after hb_cache_extend_all and before advancing.
 */
int hb_step_pack(const HbCache* cache, int n_rows, const int64_t* keys, const int* counts, const int* tokens, int n_want,
                 const int* want, int table_step, int32_t* out, int64_t capacity, int64_t* cursor, int64_t* layout);
/* Widths the block tables of a single-token step would need after growing by one token (for graph keys). */
int hb_step_decode_widths(const HbCache* cache, int n_rows, const int64_t* keys, int table_step, int* widths);
/* Attention work of a step: rows of more than token_shape_max tokens are cut into tiles (first token, count, row),
 * the tokens of shorter rows become items. Buffers need 3 * sum(ceil(count / tokens_per_tile)) and sum(counts) words. */
int hb_plan_attention(int n_rows, const int* counts, int tokens_per_tile, int token_shape_max, int* tiles, int* n_tiles, int* items,
                      int* n_items);

/* ---- scheduler ---- */
typedef struct HbScheduler HbScheduler;
/* group_windows: one entry per paged group of the cache (0 = it keeps every key); pages are reserved per group */
int hb_sched_new(int num_pages, int page_size, int n_groups, const int* group_windows, int max_seq_len, int max_batch, int max_batch_tokens,
                 int prefill_chunk_busy, int max_queue,
                 int max_in_flight, int n_eos, const int* eos, HbScheduler** out);
void hb_sched_delete(HbScheduler* s);
int hb_sched_enqueue(HbScheduler* s, int64_t key, int n_prompt, const int* prompt, int max_tokens, int ignore_eos);
/* step = -1 when there is nothing to run now */
int hb_sched_next_plan(HbScheduler* s, int* step, int* n_rows, int* n_tokens);
/* per row: key, count, sample, sampled_before, from_step, from_index; tokens: all rows' tokens in order */
int hb_sched_plan(const HbScheduler* s, int step, int64_t* keys, int* counts, int* sample, int* sampled_before, int* from_step,
                  int* from_index, int* tokens);
int hb_sched_complete(HbScheduler* s, int step, int n_sampled, const int* sampled);
int hb_sched_fail(HbScheduler* s, int step, const char* reason);
int hb_sched_cancel(HbScheduler* s, int64_t key, int* found);
/* Events since the last call: kinds 0 token, 1 finished, 2 failed. Call with capacity 0 to learn the counts
 * (events stay queued), then with room for them: reasons are written back to back, each ended by a zero byte. */
int hb_sched_take_events(HbScheduler* s, int capacity, int64_t* keys, int* kinds, int* tokens, char* reasons, int reason_capacity,
                         int* n_events, int* reason_bytes);
/* Requests whose cache must be freed; when there are more than capacity none is written and they stay queued. */
int hb_sched_take_released(HbScheduler* s, int capacity, int64_t* keys, int* n_released);
int hb_sched_state(const HbScheduler* s, int* idle, int* waiting, int* running, int* reserved_pages, int* plans_in_flight);
int hb_sched_waiting_keys(const HbScheduler* s, int64_t* keys, int capacity);

/* ---- safetensors header ----
 * Reads and checks the header of one file: it fits the file and 64 MiB, is a JSON object without a name that comes
 * twice, every tensor has a known dtype, a shape of non-negative extents and a range inside the payload of exactly
 * shape x element size bytes, and ranges do not overlap. "__metadata__" is skipped. */
typedef struct HbTensorTable HbTensorTable;
int hb_safetensors_open(const char* path, HbTensorTable** out);
void hb_safetensors_close(HbTensorTable* table);
int hb_safetensors_count(const HbTensorTable* table);
int64_t hb_safetensors_payload_start(const HbTensorTable* table);
/* name, dtype: zero-ended, owned by the table; shape: rank extents, owned by the table; begin, end: inside the payload */
int hb_safetensors_entry(const HbTensorTable* table, int index, const char** name, const char** dtype, int* rank, const int64_t** shape,
                         int64_t* begin, int64_t* end);

#ifdef __cplusplus
}
#endif
