// Host-side bookkeeping of the cache: pools of pages, a block table per request and group, request
// slots and lengths. No device code: the tensors the pages address belong to the Python layer.
//
// The reference keeps the same state in helios/crates/helios-core/src/kv/manager.rs:99-118,183-233,324-369
// (one pool, FIFO free list, growth by one page, release when a sequence ends); groups with pools of
// their own and the release of pages a window has passed are additions.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace hb {

constexpr int NO_PAGE = -1;

enum Code : int {
    OK = 0,
    OUT_OF_PAGES = 1,   // a pool or the request slots cannot give what was asked; nothing was taken
    CACHE_ERROR = 2,    // inconsistent use: unknown request, page freed twice, ...
    BAD_ARGUMENT = 3,
    BAD_STEP = 4,       // a step that is refused whole
    QUEUE_FULL = 5,
    SCHEDULER_ERROR = 6,
    BAD_FILE = 7,       // a file that is not what its name promises
};

struct Failure {
    Code code;
    std::string message;
};

// Free list of page ids with first-in first-out reuse and double-use detection.
class PagePool {
  public:
    explicit PagePool(int num_pages);
    int num_pages() const { return (int)held_.size(); }
    int available() const { return (int)free_.size(); }
    int held_count() const { return held_count_; }
    bool held(int page) const { return page >= 0 && page < num_pages() && held_[page]; }
    int take();
    void give_back(int page);
    void check() const;  // every page is either free or held, exactly once

  private:
    std::deque<int> free_;
    std::vector<uint8_t> held_;
    int held_count_ = 0;
};

struct RequestRecord {
    int slot = 0;
    int length = 0;                        // tokens whose cache entries are written
    std::vector<std::vector<int>> tables;  // per group: page of every block, NO_PAGE once a window has passed it
};

class CacheIndex {
  public:
    // windows[g] > 0: group g only ever reads the last windows[g] positions.
    CacheIndex(int page_size, int num_pages, int max_requests, std::vector<int> windows);

    int page_size() const { return page_size_; }
    int groups() const { return (int)pools_.size(); }
    int max_requests() const { return max_requests_; }
    bool has(int64_t key) const { return requests_.count(key) != 0; }
    const RequestRecord& record(int64_t key) const;
    const std::vector<int64_t>& live() const { return order_; }
    int free_pages(int group) const;
    const PagePool& pool(int group) const { return pools_.at(group); }

    int add(int64_t key);  // takes a slot; returns it
    void pages_needed(int64_t key, int new_tokens, int* out) const;
    // Gives every position of each request's next tokens a page in every group: all of them or none.
    void extend_all(int n, const int64_t* keys, const int* counts);
    // The tokens are written: moves the length and gives back the pages a window has passed.
    void advance(int64_t key, int new_tokens, std::vector<std::pair<int, int>>* released);
    void free(int64_t key);
    void check() const;

    // The most pages of one group that a request of up to `tokens` tokens can hold at any moment, when no step brings it
    // more than `largest_portion` tokens: all its blocks for a group that keeps every key (window 0), else the blocks
    // that the window behind the next position and one portion ahead of it can touch.
    static int worst_case_pages(int page_size, int window, int tokens, int largest_portion);

  private:
    RequestRecord& mutable_record(int64_t key);
    int first_needed_block(int group, int length) const;

    int page_size_, max_requests_;
    std::vector<int> windows_;
    std::vector<PagePool> pools_;
    std::unordered_map<int64_t, RequestRecord> requests_;
    std::vector<int64_t> order_;  // live requests, oldest first
    std::deque<int> free_slots_;
};

}  // namespace hb
