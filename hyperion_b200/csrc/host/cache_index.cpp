#include "cache_index.hpp"

#include <algorithm>

namespace hb {

PagePool::PagePool(int num_pages) {
    if (num_pages <= 0) throw Failure{BAD_ARGUMENT, "a page pool needs at least one page"};
    held_.assign((size_t)num_pages, 0);
    for (int page = 0; page < num_pages; ++page) free_.push_back(page);
}

int PagePool::take() {
    if (free_.empty()) throw Failure{OUT_OF_PAGES, "no free page"};
    const int page = free_.front();
    free_.pop_front();
    held_[page] = 1;
    ++held_count_;
    return page;
}

void PagePool::give_back(int page) {
    if (!held(page)) throw Failure{CACHE_ERROR, "page " + std::to_string(page) + " given back but not held"};
    held_[page] = 0;
    --held_count_;
    free_.push_back(page);
}

void PagePool::check() const {
    std::vector<uint8_t> seen(held_.size(), 0);
    for (int page : free_) {
        if (page < 0 || page >= num_pages() || seen[page] || held_[page]) throw Failure{CACHE_ERROR, "page accounting broken"};
        seen[page] = 1;
    }
    int held = 0;
    for (uint8_t flag : held_) held += flag;
    if (held != held_count_ || (int)free_.size() + held != num_pages()) throw Failure{CACHE_ERROR, "page accounting broken"};
}

CacheIndex::CacheIndex(int page_size, int num_pages, int max_requests, std::vector<int> windows)
    : page_size_(page_size), max_requests_(max_requests), windows_(std::move(windows)) {
    if (page_size <= 0 || (page_size & (page_size - 1)))
        throw Failure{BAD_ARGUMENT, "page_size must be a power of two, got " + std::to_string(page_size)};
    if (max_requests < 0) throw Failure{BAD_ARGUMENT, "max_requests must not be negative"};
    for (size_t g = 0; g < windows_.size(); ++g) pools_.emplace_back(num_pages);
    for (int slot = 0; slot < max_requests; ++slot) free_slots_.push_back(slot);
}

const RequestRecord& CacheIndex::record(int64_t key) const {
    auto found = requests_.find(key);
    if (found == requests_.end()) throw Failure{CACHE_ERROR, "unknown request"};
    return found->second;
}

RequestRecord& CacheIndex::mutable_record(int64_t key) {
    auto found = requests_.find(key);
    if (found == requests_.end()) throw Failure{CACHE_ERROR, "unknown request"};
    return found->second;
}

int CacheIndex::free_pages(int group) const {
    if (pools_.empty()) return 0;
    if (group < 0 || group >= groups()) throw Failure{BAD_ARGUMENT, "no such group"};
    return pools_[group].available();
}

int CacheIndex::add(int64_t key) {
    if (has(key)) throw Failure{CACHE_ERROR, "the request is already live"};
    if (free_slots_.empty()) throw Failure{OUT_OF_PAGES, "all " + std::to_string(max_requests_) + " request slots are taken"};
    RequestRecord record;
    record.slot = free_slots_.front();
    free_slots_.pop_front();
    record.tables.resize(pools_.size());
    requests_.emplace(key, std::move(record));
    order_.push_back(key);
    return requests_[key].slot;
}

int CacheIndex::first_needed_block(int group, int length) const {
    // the first block a query at position `length` (the next one) can still read
    const int window = windows_[group];
    if (window <= 0) return 0;
    return std::max(0, length - window + 1) / page_size_;
}

int CacheIndex::worst_case_pages(int page_size, int window, int tokens, int largest_portion) {
    if (page_size < 1 || window < 0 || tokens < 0 || largest_portion < 1) throw Failure{BAD_ARGUMENT, "worst_case_pages: bad sizes"};
    const long long all = ((long long)tokens + page_size - 1) / page_size;
    if (window == 0) return (int)all;
    // before a step the table holds blocks from first_needed_block(length) on; the step adds blocks up to its last token:
    // ceil((a + window - 1 + n) / page) - floor(a / page) <= ceil((window + n - 1) / page) + 1 for every start a
    const long long spanned = ((long long)window + largest_portion - 1 + page_size - 1) / page_size + 1;
    return (int)std::min(all, spanned);
}

void CacheIndex::pages_needed(int64_t key, int new_tokens, int* out) const {
    const RequestRecord& r = record(key);
    const int blocks = (r.length + new_tokens + page_size_ - 1) / page_size_;
    for (int g = 0; g < groups(); ++g) out[g] = std::max(0, blocks - (int)r.tables[g].size());
}

void CacheIndex::extend_all(int n, const int64_t* keys, const int* counts) {
    std::vector<int> totals(pools_.size(), 0), need(pools_.size(), 0);
    for (int i = 0; i < n; ++i) {
        pages_needed(keys[i], counts[i], need.data());
        for (int g = 0; g < groups(); ++g) totals[g] += need[g];
    }
    for (int g = 0; g < groups(); ++g)
        if (totals[g] > pools_[g].available())
            throw Failure{OUT_OF_PAGES, "the step needs " + std::to_string(totals[g]) + " more pages, " + std::to_string(pools_[g].available()) + " free"};
    for (int i = 0; i < n; ++i) {
        RequestRecord& r = mutable_record(keys[i]);
        pages_needed(keys[i], counts[i], need.data());  // again: the same request may stand twice in the list
        for (int g = 0; g < groups(); ++g)
            for (int p = 0; p < need[g]; ++p) r.tables[g].push_back(pools_[g].take());
    }
}

void CacheIndex::advance(int64_t key, int new_tokens, std::vector<std::pair<int, int>>* released) {
    RequestRecord& r = mutable_record(key);
    for (int g = 0; g < groups(); ++g)
        if ((long long)r.tables[g].size() * page_size_ < (long long)r.length + new_tokens)
            throw Failure{CACHE_ERROR, "the request advanced past its pages"};
    r.length += new_tokens;
    for (int g = 0; g < groups(); ++g) {
        std::vector<int>& table = r.tables[g];
        const int passed = std::min(first_needed_block(g, r.length), (int)table.size());
        for (int block = 0; block < passed; ++block) {
            if (table[block] == NO_PAGE) continue;
            pools_[g].give_back(table[block]);
            if (released) released->emplace_back(g, table[block]);
            table[block] = NO_PAGE;
        }
    }
}

void CacheIndex::free(int64_t key) {
    auto found = requests_.find(key);
    if (found == requests_.end()) throw Failure{CACHE_ERROR, "the request is not live"};
    for (int g = 0; g < groups(); ++g)
        for (int page : found->second.tables[g])
            if (page != NO_PAGE) pools_[g].give_back(page);
    free_slots_.push_back(found->second.slot);
    requests_.erase(found);
    order_.erase(std::find(order_.begin(), order_.end(), key));
}

void CacheIndex::check() const {
    for (int g = 0; g < groups(); ++g) {
        pools_[g].check();
        std::vector<uint8_t> seen((size_t)pools_[g].num_pages(), 0);
        int in_tables = 0;
        for (const auto& item : requests_)
            for (int page : item.second.tables[g]) {
                if (page == NO_PAGE) continue;
                if (page < 0 || page >= pools_[g].num_pages() || seen[page]) throw Failure{CACHE_ERROR, "page " + std::to_string(page) + " is in two tables"};
                if (!pools_[g].held(page)) throw Failure{CACHE_ERROR, "held pages and tables disagree"};
                seen[page] = 1;
                ++in_tables;
            }
        if (in_tables != pools_[g].held_count()) throw Failure{CACHE_ERROR, "held pages and tables disagree"};
    }
    std::vector<uint8_t> slots((size_t)max_requests_, 0);
    size_t count = 0;
    for (const auto& item : requests_) {
        const int slot = item.second.slot;
        if (slot < 0 || slot >= max_requests_ || slots[slot]) throw Failure{CACHE_ERROR, "slot accounting broken"};
        slots[slot] = 1;
        ++count;
    }
    for (int slot : free_slots_) {
        if (slot < 0 || slot >= max_requests_ || slots[slot]) throw Failure{CACHE_ERROR, "slot accounting broken"};
        slots[slot] = 1;
        ++count;
    }
    if (count != (size_t)max_requests_ || order_.size() != requests_.size()) throw Failure{CACHE_ERROR, "slot accounting broken"};
}

}  // namespace hb
