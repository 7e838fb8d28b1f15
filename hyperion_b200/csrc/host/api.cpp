// The C interface over the C++ classes: catches failures, keeps the last error text per thread.
#include "runtime.h"

#include <algorithm>
#include <cstring>
#include <new>
#include <string>

#include "cache_index.hpp"
#include "safetensors.hpp"
#include "scheduler.hpp"

#define HB_API extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string last_error;

template <typename F>
int guarded(F&& body) {
    try {
        body();
        return HB_HOST_OK;
    } catch (const hb::Failure& failure) {
        last_error = failure.message;
        return (int)failure.code;
    } catch (const std::bad_alloc&) {
        last_error = "out of host memory";
        return HB_HOST_BAD_ARGUMENT;
    } catch (const std::exception& error) {
        last_error = error.what();
        return HB_HOST_BAD_ARGUMENT;
    }
}

void require(bool condition, const char* message) {
    if (!condition) throw hb::Failure{hb::BAD_ARGUMENT, message};
}
}  // namespace

struct HbPool { hb::PagePool pool; };
struct HbCache { hb::CacheIndex index; };
struct HbScheduler {
    hb::Scheduler scheduler;
    std::vector<hb::Event> events;   // taken from the scheduler, not yet handed out
    std::vector<int64_t> released;  // likewise
};

HB_API const char* hb_host_last_error(void) { return last_error.c_str(); }

// ---------------------------------------------------------------- pool
HB_API int hb_pool_new(int num_pages, HbPool** out) {
    return guarded([&] { *out = new HbPool{hb::PagePool(num_pages)}; });
}
HB_API void hb_pool_delete(HbPool* pool) { delete pool; }
HB_API int hb_pool_available(const HbPool* pool) { return pool->pool.available(); }
HB_API int hb_pool_take(HbPool* pool, int* page) {
    return guarded([&] { *page = pool->pool.take(); });
}
HB_API int hb_pool_give_back(HbPool* pool, int page) {
    return guarded([&] { pool->pool.give_back(page); });
}
HB_API int hb_pool_is_held(const HbPool* pool, int page) { return pool->pool.held(page) ? 1 : 0; }
HB_API int hb_pool_check(const HbPool* pool) {
    return guarded([&] { pool->pool.check(); });
}

// ---------------------------------------------------------------- cache index
HB_API int hb_cache_new(int page_size, int num_pages, int max_requests, int n_groups, const int* windows, HbCache** out) {
    return guarded([&] {
        require(n_groups >= 0, "the number of groups must not be negative");
        *out = new HbCache{hb::CacheIndex(page_size, num_pages, max_requests, std::vector<int>(windows, windows + n_groups))};
    });
}
HB_API void hb_cache_delete(HbCache* cache) { delete cache; }
HB_API int hb_cache_has(const HbCache* cache, int64_t key) { return cache->index.has(key) ? 1 : 0; }
HB_API int hb_cache_add(HbCache* cache, int64_t key, int* slot) {
    return guarded([&] { *slot = cache->index.add(key); });
}
HB_API int hb_cache_length(const HbCache* cache, int64_t key, int* length) {
    return guarded([&] { *length = cache->index.record(key).length; });
}
HB_API int hb_cache_slot(const HbCache* cache, int64_t key, int* slot) {
    return guarded([&] { *slot = cache->index.record(key).slot; });
}
HB_API int hb_cache_table_size(const HbCache* cache, int group, int64_t key, int* size) {
    return guarded([&] {
        require(group >= 0 && group < cache->index.groups(), "no such group");
        *size = (int)cache->index.record(key).tables[group].size();
    });
}
HB_API int hb_cache_table(const HbCache* cache, int group, int64_t key, int* pages, int capacity) {
    return guarded([&] {
        require(group >= 0 && group < cache->index.groups(), "no such group");
        const std::vector<int>& table = cache->index.record(key).tables[group];
        require((int)table.size() <= capacity, "the table does not fit the buffer");
        std::copy(table.begin(), table.end(), pages);
    });
}
HB_API int hb_cache_pages_needed(const HbCache* cache, int64_t key, int new_tokens, int* per_group) {
    return guarded([&] { cache->index.pages_needed(key, new_tokens, per_group); });
}
HB_API int hb_cache_extend_all(HbCache* cache, int n, const int64_t* keys, const int* counts) {
    return guarded([&] { cache->index.extend_all(n, keys, counts); });
}
HB_API int hb_cache_advance(HbCache* cache, int64_t key, int new_tokens, int* released, int capacity, int* n_released) {
    return guarded([&] {
        std::vector<std::pair<int, int>> pairs;
        cache->index.advance(key, new_tokens, &pairs);
        if (n_released) *n_released = (int)pairs.size();
        for (int i = 0; i < (int)pairs.size() && i < capacity; ++i) {
            released[2 * i] = pairs[i].first;
            released[2 * i + 1] = pairs[i].second;
        }
    });
}
HB_API int hb_cache_advance_all(HbCache* cache, int n, const int64_t* keys, const int* counts) {
    return guarded([&] {
        for (int i = 0; i < n; ++i) cache->index.advance(keys[i], counts[i], nullptr);
    });
}
HB_API int hb_cache_free(HbCache* cache, int64_t key) {
    return guarded([&] { cache->index.free(key); });
}
HB_API int hb_cache_free_pages(const HbCache* cache, int group, int* pages) {
    return guarded([&] { *pages = cache->index.free_pages(group); });
}
HB_API int hb_cache_live(const HbCache* cache, int64_t* keys, int capacity, int* n_live) {
    return guarded([&] {
        const std::vector<int64_t>& live = cache->index.live();
        *n_live = (int)live.size();
        for (int i = 0; i < (int)live.size() && i < capacity; ++i) keys[i] = live[i];
    });
}
HB_API int hb_cache_lengths(const HbCache* cache, int n, const int64_t* keys, int* lengths, int* slots) {
    return guarded([&] {
        for (int i = 0; i < n; ++i) {
            if (cache->index.has(keys[i])) {
                const hb::RequestRecord& r = cache->index.record(keys[i]);
                lengths[i] = r.length;
                slots[i] = r.slot;
            } else {
                lengths[i] = -1;
                slots[i] = -1;
            }
        }
    });
}
HB_API int hb_cache_check(const HbCache* cache) {
    return guarded([&] { cache->index.check(); });
}
HB_API int hb_cache_worst_case_pages(int page_size, int window, int tokens, int largest_portion, int* pages) {
    return guarded([&] { *pages = hb::CacheIndex::worst_case_pages(page_size, window, tokens, largest_portion); });
}

// ---------------------------------------------------------------- step assembly
namespace {
int64_t aligned(int64_t words) { return (words + 3) & ~(int64_t)3; }

int table_width(const hb::CacheIndex& index, int group, int n_rows, const int64_t* keys, int table_step, int extra_tokens) {
    int width = 1;
    for (int r = 0; r < n_rows; ++r) {
        const hb::RequestRecord& record = index.record(keys[r]);
        int blocks = (int)record.tables[group].size();
        if (extra_tokens) blocks = std::max(blocks, (record.length + extra_tokens + index.page_size() - 1) / index.page_size());
        width = std::max(width, blocks);
    }
    if (table_step > 0) width = (width + table_step - 1) / table_step * table_step;
    if (table_step < 0) {  // the next power of two, at least -table_step: few distinct widths over a long context
        int rounded = -table_step;
        while (rounded < width) rounded *= 2;
        width = rounded;
    }
    return width;
}
}  // namespace

HB_API int hb_step_pack(const HbCache* cache, int n_rows, const int64_t* keys, const int* counts, const int* tokens, int n_want,
                        const int* want, int table_step, int32_t* out, int64_t capacity, int64_t* cursor, int64_t* layout) {
    return guarded([&] {
        const hb::CacheIndex& index = cache->index;
        require(n_rows > 0 && n_want >= 0, "a step needs at least one row");
        int64_t total = 0;
        for (int r = 0; r < n_rows; ++r) {
            require(counts[r] > 0, "a row brings no tokens");
            total += counts[r];
        }
        const int groups = index.groups();
        std::vector<int> widths((size_t)groups);
        for (int g = 0; g < groups; ++g) widths[g] = table_width(index, g, n_rows, keys, table_step, 0);
        int64_t need = *cursor;
        need = aligned(need) + total;  // token ids
        need = aligned(need) + total;  // positions
        need = aligned(need) + total;  // rows
        need = aligned(need) + n_rows + 1;
        need = aligned(need) + n_rows;
        need = aligned(need) + n_want;
        for (int g = 0; g < groups; ++g) need = aligned(need) + (int64_t)n_rows * widths[g];
        if (need > capacity) throw hb::Failure{hb::BAD_ARGUMENT, "the step's metadata needs " + std::to_string(need) + " words"};

        int64_t at = *cursor;
        int array = 0;
        auto begin = [&](int64_t count, int64_t rows, int64_t columns) {
            at = aligned(at);
            layout[4 * array] = at;
            layout[4 * array + 1] = count;
            layout[4 * array + 2] = rows;
            layout[4 * array + 3] = columns;
            ++array;
            int32_t* where = out + at;
            at += count;
            return where;
        };
        int32_t* token_ids = begin(total, total, 1);
        std::memcpy(token_ids, tokens, sizeof(int32_t) * (size_t)total);
        int32_t* positions = begin(total, total, 1);
        int32_t* token_row = begin(total, total, 1);
        int32_t* row_start = begin(n_rows + 1, n_rows + 1, 1);
        int32_t* slots = begin(n_rows, n_rows, 1);
        int64_t t = 0;
        for (int r = 0; r < n_rows; ++r) {
            const hb::RequestRecord& record = index.record(keys[r]);
            row_start[r] = (int32_t)t;
            slots[r] = record.slot;
            for (int i = 0; i < counts[r]; ++i, ++t) {
                positions[t] = record.length + i;
                token_row[t] = r;
            }
        }
        row_start[n_rows] = (int32_t)total;
        int32_t* wanted = begin(n_want, n_want, 1);
        for (int i = 0; i < n_want; ++i) {
            require(want[i] >= 0 && want[i] < total, "a wanted place is outside the step's tokens");
            wanted[i] = want[i];
        }
        for (int g = 0; g < groups; ++g) {
            int32_t* table = begin((int64_t)n_rows * widths[g], n_rows, widths[g]);
            for (int r = 0; r < n_rows; ++r) {
                const std::vector<int>& pages = index.record(keys[r]).tables[g];
                int32_t* row = table + (int64_t)r * widths[g];
                std::copy(pages.begin(), pages.end(), row);
                std::fill(row + pages.size(), row + widths[g], hb::NO_PAGE);
            }
        }
        *cursor = at;
    });
}

HB_API int hb_step_decode_widths(const HbCache* cache, int n_rows, const int64_t* keys, int table_step, int* widths) {
    return guarded([&] {
        for (int g = 0; g < cache->index.groups(); ++g) widths[g] = table_width(cache->index, g, n_rows, keys, table_step, 1);
    });
}

HB_API int hb_plan_attention(int n_rows, const int* counts, int tokens_per_tile, int token_shape_max, int* tiles, int* n_tiles, int* items,
                             int* n_items) {
    return guarded([&] {
        require(tokens_per_tile > 0, "tokens_per_tile must be positive");
        int start = 0, t = 0, it = 0;
        for (int r = 0; r < n_rows; ++r) {
            if (counts[r] <= token_shape_max) {
                for (int i = 0; i < counts[r]; ++i) items[it++] = start + i;
            } else {
                for (int first = 0; first < counts[r]; first += tokens_per_tile) {
                    tiles[3 * t] = start + first;
                    tiles[3 * t + 1] = std::min(tokens_per_tile, counts[r] - first);
                    tiles[3 * t + 2] = r;
                    ++t;
                }
            }
            start += counts[r];
        }
        *n_tiles = t;
        *n_items = it;
    });
}

// ---------------------------------------------------------------- scheduler
HB_API int hb_sched_new(int num_pages, int page_size, int n_groups, const int* group_windows, int max_seq_len, int max_batch, int max_batch_tokens,
                        int prefill_chunk_busy, int max_queue, int max_in_flight, int n_eos, const int* eos, HbScheduler** out) {
    return guarded([&] {
        if (n_groups < 0) throw hb::Failure{hb::BAD_ARGUMENT, "n_groups must not be negative"};
        hb::SchedulerConfig config;
        config.num_pages = num_pages;
        config.group_windows.assign(group_windows, group_windows + n_groups);
        config.page_size = page_size;
        config.max_seq_len = max_seq_len;
        config.max_batch = max_batch;
        config.max_batch_tokens = max_batch_tokens;
        config.prefill_chunk_busy = prefill_chunk_busy;
        config.max_queue = max_queue;
        config.max_in_flight = max_in_flight;
        config.eos_token_ids.assign(eos, eos + n_eos);
        *out = new HbScheduler{hb::Scheduler(std::move(config)), {}, {}};
    });
}
HB_API void hb_sched_delete(HbScheduler* s) { delete s; }
HB_API int hb_sched_enqueue(HbScheduler* s, int64_t key, int n_prompt, const int* prompt, int max_tokens, int ignore_eos) {
    return guarded([&] { s->scheduler.enqueue(key, std::vector<int>(prompt, prompt + n_prompt), max_tokens, ignore_eos != 0); });
}
HB_API int hb_sched_next_plan(HbScheduler* s, int* step, int* n_rows, int* n_tokens) {
    return guarded([&] {
        const hb::Plan* plan = s->scheduler.next_plan();
        *step = plan ? plan->step : -1;
        *n_rows = plan ? (int)plan->rows.size() : 0;
        int tokens = 0;
        if (plan)
            for (const hb::PlanRow& row : plan->rows) tokens += (int)row.tokens.size();
        *n_tokens = tokens;
    });
}
HB_API int hb_sched_plan(const HbScheduler* s, int step, int64_t* keys, int* counts, int* sample, int* sampled_before, int* from_step,
                         int* from_index, int* tokens) {
    return guarded([&] {
        const hb::Plan* plan = s->scheduler.in_flight(step);
        if (!plan) throw hb::Failure{hb::SCHEDULER_ERROR, "no such plan in flight"};
        int t = 0;
        for (size_t r = 0; r < plan->rows.size(); ++r) {
            const hb::PlanRow& row = plan->rows[r];
            keys[r] = row.key;
            counts[r] = (int)row.tokens.size();
            sample[r] = row.sample ? 1 : 0;
            sampled_before[r] = row.sampled_before;
            from_step[r] = row.from_step;
            from_index[r] = row.from_index;
            for (int token : row.tokens) tokens[t++] = token;
        }
    });
}
HB_API int hb_sched_complete(HbScheduler* s, int step, int n_sampled, const int* sampled) {
    return guarded([&] { s->scheduler.complete(step, n_sampled, sampled); });
}
HB_API int hb_sched_fail(HbScheduler* s, int step, const char* reason) {
    return guarded([&] { s->scheduler.fail(step, reason ? reason : ""); });
}
HB_API int hb_sched_cancel(HbScheduler* s, int64_t key, int* found) {
    return guarded([&] { *found = s->scheduler.cancel(key) ? 1 : 0; });
}
HB_API int hb_sched_take_events(HbScheduler* s, int capacity, int64_t* keys, int* kinds, int* tokens, char* reasons, int reason_capacity,
                                int* n_events, int* reason_bytes) {
    return guarded([&] {
        std::vector<hb::Event> fresh = s->scheduler.take_events();
        s->events.insert(s->events.end(), fresh.begin(), fresh.end());
        int bytes = 0;
        for (const hb::Event& e : s->events) bytes += (int)e.reason.size() + 1;
        *n_events = (int)s->events.size();
        *reason_bytes = bytes;
        if (capacity < (int)s->events.size() || reason_capacity < bytes) return;  // the caller asks again with room
        int at = 0;
        for (size_t i = 0; i < s->events.size(); ++i) {
            const hb::Event& e = s->events[i];
            keys[i] = e.key;
            kinds[i] = e.kind;
            tokens[i] = e.token;
            std::memcpy(reasons + at, e.reason.c_str(), e.reason.size() + 1);
            at += (int)e.reason.size() + 1;
        }
        s->events.clear();
    });
}
HB_API int hb_sched_take_released(HbScheduler* s, int capacity, int64_t* keys, int* n_released) {
    return guarded([&] {
        std::vector<int64_t> fresh = s->scheduler.take_released();
        s->released.insert(s->released.end(), fresh.begin(), fresh.end());
        *n_released = (int)s->released.size();
        if (capacity < (int)s->released.size()) return;  // the caller asks again with room
        std::copy(s->released.begin(), s->released.end(), keys);
        s->released.clear();
    });
}
HB_API int hb_sched_state(const HbScheduler* s, int* idle, int* waiting, int* running, int* reserved_pages, int* plans_in_flight) {
    return guarded([&] {
        *idle = s->scheduler.idle() ? 1 : 0;
        *waiting = s->scheduler.waiting();
        *running = s->scheduler.running();
        *reserved_pages = s->scheduler.reserved_pages();
        *plans_in_flight = s->scheduler.plans_in_flight();
    });
}
HB_API int hb_sched_waiting_keys(const HbScheduler* s, int64_t* keys, int capacity) {
    return guarded([&] {
        std::vector<int64_t> waiting = s->scheduler.waiting_keys();
        require((int)waiting.size() <= capacity, "room for fewer waiting requests than there are");
        std::copy(waiting.begin(), waiting.end(), keys);
    });
}

// ---------------------------------------------------------------- safetensors header
struct HbTensorTable { hb::TensorTable table; };

HB_API int hb_safetensors_open(const char* path, HbTensorTable** out) {
    return guarded([&] {
        require(path != nullptr && out != nullptr, "hb_safetensors_open: null argument");
        *out = new HbTensorTable{hb::read_safetensors_header(path)};
    });
}
HB_API void hb_safetensors_close(HbTensorTable* table) { delete table; }
HB_API int hb_safetensors_count(const HbTensorTable* table) { return (int)table->table.tensors.size(); }
HB_API int64_t hb_safetensors_payload_start(const HbTensorTable* table) { return table->table.payload_start; }
HB_API int hb_safetensors_entry(const HbTensorTable* table, int index, const char** name, const char** dtype, int* rank, const int64_t** shape,
                                int64_t* begin, int64_t* end) {
    return guarded([&] {
        require(index >= 0 && index < (int)table->table.tensors.size(), "hb_safetensors_entry: no such tensor");
        const hb::TensorRecord& record = table->table.tensors[(size_t)index];
        *name = record.name.c_str();
        *dtype = record.dtype.c_str();
        *rank = (int)record.shape.size();
        *shape = record.shape.data();
        *begin = record.begin;
        *end = record.end;
    });
}
