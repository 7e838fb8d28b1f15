// The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
// finishes and releases. A state machine without clock, thread or device: the same trace of
// requests always yields the same plans (as helios/crates/helios-core/src/step_scheduler.rs:92-154).
//
// Policies kept from the reference: a bounded first-in first-out queue (step_scheduler.rs:113-124);
// admission by worst-case reservation of pages, so pages never run out under a running request and
// nothing is preempted (step_scheduler.rs:160-201); the oldest prompt first, with smaller portions
// while requests are decoding (step_scheduler.rs:206-213,238-241); an end-of-sequence token ends a
// request and is not emitted (step_scheduler.rs:364-383); when more requests decode than the step's
// token budget holds, they take turns from a cursor that moves on, so none starves
// (step_scheduler.rs:273-289). Unlike the reference a step mixes decode
// rows and prompt portions, and plans may be made before the results of the plans before them are
// in: a row whose token is still on the device carries PENDING_TOKEN and names where it comes from.
// Pages are reserved per group of the cache: a group that keeps every key costs a request the pages
// of its whole length, a windowed group the pages its window and one portion can span, and a model
// without paged groups costs none (CacheIndex::worst_case_pages).
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_index.hpp"

namespace hb {

constexpr int PENDING_TOKEN = -1;

struct SchedulerConfig {
    int num_pages = 0;             // pages in the pool of every paged group
    int page_size = 1;
    std::vector<int> group_windows{0};  // one entry per paged group of the cache: 0 = keeps every key, else its window
    int max_seq_len = 0;
    int max_batch = 64;            // most requests live at a time
    int max_batch_tokens = 2048;   // token budget of one step
    int prefill_chunk_busy = 512;  // largest prompt portion while requests are decoding
    int max_queue = 1 << 16;
    int max_in_flight = 1;         // plans that may be made before the oldest one's results are in
    std::vector<int> eos_token_ids;
};

struct PlanRow {
    int64_t key = 0;
    std::vector<int> tokens;
    bool sample = false;     // the row's last token ends the prompt or is a decode token: a token is chosen after it
    int sampled_before = 0;  // tokens the request has sampled so far (the draw counter)
    int from_step = -1;      // tokens == {PENDING_TOKEN}: the plan ...
    int from_index = -1;     // ... and the index among its sampled rows the token comes from
};

struct Plan {
    int step = -1;
    std::vector<PlanRow> rows;
};

enum EventKind : int { EVENT_TOKEN = 0, EVENT_FINISHED = 1, EVENT_FAILED = 2 };

struct Event {
    int64_t key;
    int kind;
    int token;           // EVENT_TOKEN
    std::string reason;  // "stop" | "length" | "cancelled" | the text of a failure
};

class Scheduler {
  public:
    explicit Scheduler(SchedulerConfig config);

    void enqueue(int64_t key, std::vector<int> prompt, int max_tokens, bool ignore_eos);
    // The next step; nullptr when there is nothing to run now. The plan stays valid until it is completed or failed.
    const Plan* next_plan();
    const Plan* in_flight(int step) const;
    void complete(int step, int n_sampled, const int* sampled);  // the oldest plan in flight; sampled in row order
    void fail(int step, const std::string& reason);                // any plan in flight: its requests fail and are released
    bool cancel(int64_t key);

    std::vector<Event> take_events();
    std::vector<int64_t> take_released();
    bool idle() const { return waiting_.empty() && running_.empty(); }
    int reserved_pages() const;  // of the group that has reserved most
    int waiting() const { return (int)waiting_.size(); }
    int running() const { return (int)running_.size(); }
    int plans_in_flight() const { return (int)in_flight_.size(); }
    std::vector<int64_t> waiting_keys() const;
    std::vector<int64_t> running_keys() const { return order_; }

  private:
    struct Request {
        int64_t key;
        std::vector<int> prompt;
        int max_tokens;
        bool ignore_eos;
    };
    struct Sequence {
        Request request;
        std::vector<int> reserved_pages;  // per paged group
        int fed = 0;              // prompt tokens already planned
        int planned_samples = 0;  // sampled rows planned so far, results in or not
        int generated = 0;        // tokens whose values are in
        // what the next decode row feeds: nothing, a token, or a place in a plan in flight
        enum Feed { NONE, TOKEN, PLACE } feed = NONE;
        int feed_token = 0, feed_step = -1, feed_index = -1;
        bool prefilling() const { return fed < (int)request.prompt.size(); }
    };

    std::vector<int> reserved_per_group() const;
    void admit();
    void finish(int64_t key, const char* reason);
    void drop(int64_t key);

    SchedulerConfig config_;
    std::deque<Request> waiting_;
    std::unordered_map<int64_t, Sequence> running_;
    std::vector<int64_t> order_;  // running requests in admission order
    std::vector<Event> events_;
    std::vector<int64_t> released_;
    std::deque<Plan> in_flight_;  // oldest first
    int step_ = 0;
    size_t decode_cursor_ = 0;  // index into order_ where the next step's decode rows start
};

}  // namespace hb
