#include "scheduler.hpp"

#include <algorithm>

namespace hb {

Scheduler::Scheduler(SchedulerConfig config) : config_(std::move(config)) {
    if (config_.max_batch_tokens < 1 || config_.prefill_chunk_busy < 1 || config_.max_batch < 1)
        throw Failure{BAD_ARGUMENT, "max_batch_tokens, prefill_chunk_busy and max_batch must be at least 1"};
    if (config_.page_size < 1 || config_.max_in_flight < 1) throw Failure{BAD_ARGUMENT, "page_size and max_in_flight must be at least 1"};
    for (int window : config_.group_windows)
        if (window < 0) throw Failure{BAD_ARGUMENT, "a group's window must not be negative"};
}

void Scheduler::enqueue(int64_t key, std::vector<int> prompt, int max_tokens, bool ignore_eos) {
    if ((int)waiting_.size() >= config_.max_queue) throw Failure{QUEUE_FULL, std::to_string(waiting_.size()) + " requests are waiting"};
    if (max_tokens < 1) throw Failure{BAD_ARGUMENT, "max_tokens must be at least 1"};
    if (running_.count(key)) throw Failure{BAD_ARGUMENT, "the request id is already known"};
    for (const Request& r : waiting_)
        if (r.key == key) throw Failure{BAD_ARGUMENT, "the request id is already known"};
    waiting_.push_back(Request{key, std::move(prompt), max_tokens, ignore_eos});
}

std::vector<int> Scheduler::reserved_per_group() const {
    std::vector<int> totals(config_.group_windows.size(), 0);
    for (const auto& item : running_)
        for (size_t g = 0; g < totals.size(); ++g) totals[g] += item.second.reserved_pages[g];
    return totals;
}

int Scheduler::reserved_pages() const {
    int most = 0;
    for (int total : reserved_per_group()) most = std::max(most, total);
    return most;
}

std::vector<int64_t> Scheduler::waiting_keys() const {
    std::vector<int64_t> keys;
    for (const Request& r : waiting_) keys.push_back(r.key);
    return keys;
}

void Scheduler::admit() {
    const SchedulerConfig& c = config_;
    const size_t groups = c.group_windows.size();
    std::vector<int> reserved = reserved_per_group(), need(groups, 0);
    while (!waiting_.empty() && (int)running_.size() < c.max_batch) {
        Request& request = waiting_.front();
        const int prompt = (int)request.prompt.size();
        if (prompt == 0 || prompt >= c.max_seq_len) {
            events_.push_back(Event{request.key, EVENT_FAILED, 0,
                                    "prompt of " + std::to_string(prompt) + " tokens is outside 1.." + std::to_string(c.max_seq_len - 1)});
            waiting_.pop_front();
            continue;
        }
        // the request's greatest length, in 64 bits: max_tokens may be anything up to INT_MAX
        const int tokens = (int)std::min<long long>((long long)prompt + request.max_tokens, c.max_seq_len);
        const int portion = std::max(1, std::min(prompt, c.max_batch_tokens));  // the largest portion a step can bring
        int most = 0;
        bool fits = true;
        for (size_t g = 0; g < groups; ++g) {
            need[g] = CacheIndex::worst_case_pages(c.page_size, c.group_windows[g], tokens, portion);
            most = std::max(most, need[g]);
            fits = fits && reserved[g] + need[g] <= c.num_pages;
        }
        if (most > c.num_pages) {
            events_.push_back(Event{request.key, EVENT_FAILED, 0,
                                    "needs " + std::to_string(most) + " pages, the pool has " + std::to_string(c.num_pages)});
            waiting_.pop_front();
            continue;
        }
        if (!fits) return;  // waits for running requests to finish; order is kept
        Sequence s;
        s.request = std::move(request);
        s.reserved_pages = need;
        const int64_t key = s.request.key;
        waiting_.pop_front();
        running_.emplace(key, std::move(s));
        order_.push_back(key);
        for (size_t g = 0; g < groups; ++g) reserved[g] += need[g];
    }
}

const Plan* Scheduler::next_plan() {
    if ((int)in_flight_.size() >= config_.max_in_flight) throw Failure{SCHEDULER_ERROR, "the previous plan has not been completed"};
    admit();
    const SchedulerConfig& c = config_;
    Plan plan;
    int budget = c.max_batch_tokens;
    bool decoding = false;
    // Decode rows start at the cursor and wrap around; when the budget ends before every decoding request had its
    // row, the next step starts behind the last one served, so that they take turns (the reference's round robin
    // over its largest bucket, step_scheduler.rs:273-289). The plan keeps admission order among the rows it holds.
    const size_t n = order_.size();
    if (decode_cursor_ >= n) decode_cursor_ = 0;
    // Prompts that wait keep up to half of the budget, so that decoding requests alone cannot shut a newcomer out.
    long long prompt_tokens = 0;
    for (int64_t key : order_) {
        const Sequence& s = running_.at(key);
        prompt_tokens += (long long)s.request.prompt.size() - s.fed;
    }
    const int decode_budget = std::max(1, budget - (int)std::min<long long>(budget / 2, prompt_tokens));
    std::vector<size_t> chosen;
    bool skipped = false;
    size_t last = 0;
    for (size_t k = 0; k < n; ++k) {
        const size_t at = (decode_cursor_ + k) % n;
        if (running_.at(order_[at]).feed == Sequence::NONE) continue;
        decoding = true;
        if ((int)chosen.size() == decode_budget) { skipped = true; continue; }
        chosen.push_back(at);
        last = at;
    }
    decode_cursor_ = skipped ? (last + 1) % n : 0;
    std::sort(chosen.begin(), chosen.end());
    for (size_t at : chosen) {
        const int64_t key = order_[at];
        Sequence& s = running_.at(key);
        PlanRow row;
        row.key = key;
        row.sample = true;
        row.sampled_before = s.planned_samples;
        if (s.feed == Sequence::PLACE) {
            row.tokens = {PENDING_TOKEN};
            row.from_step = s.feed_step;
            row.from_index = s.feed_index;
        } else {
            row.tokens = {s.feed_token};
        }
        plan.rows.push_back(std::move(row));
        --budget;
    }
    const int limit = decoding ? c.prefill_chunk_busy : c.max_batch_tokens;
    for (int64_t key : order_) {
        if (budget == 0) break;
        Sequence& s = running_.at(key);
        if (!s.prefilling()) continue;
        const std::vector<int>& prompt = s.request.prompt;
        const int count = std::min({(int)prompt.size() - s.fed, budget, limit});
        PlanRow row;
        row.key = key;
        row.tokens.assign(prompt.begin() + s.fed, prompt.begin() + s.fed + count);
        row.sample = s.fed + count == (int)prompt.size();
        row.sampled_before = 0;
        plan.rows.push_back(std::move(row));
        s.fed += count;
        budget -= count;
    }
    if (plan.rows.empty()) return nullptr;
    plan.step = step_++;
    int sampled = 0;
    for (const PlanRow& row : plan.rows) {  // what each request feeds next is known now, but for the token's value
        if (!row.sample) continue;
        Sequence& s = running_.at(row.key);
        ++s.planned_samples;
        const bool more = s.planned_samples < s.request.max_tokens && (int)s.request.prompt.size() + s.planned_samples < c.max_seq_len;
        s.feed = more ? Sequence::PLACE : Sequence::NONE;
        s.feed_step = plan.step;
        s.feed_index = sampled++;
    }
    in_flight_.push_back(std::move(plan));
    return &in_flight_.back();
}

const Plan* Scheduler::in_flight(int step) const {
    for (const Plan& plan : in_flight_)
        if (plan.step == step) return &plan;
    return nullptr;
}

void Scheduler::drop(int64_t key) {
    running_.erase(key);
    const auto found = std::find(order_.begin(), order_.end(), key);
    if ((size_t)(found - order_.begin()) < decode_cursor_) --decode_cursor_;  // the cursor stays on the same request
    order_.erase(found);
    released_.push_back(key);
}

void Scheduler::finish(int64_t key, const char* reason) {
    drop(key);
    events_.push_back(Event{key, EVENT_FINISHED, 0, reason});
}

void Scheduler::complete(int step, int n_sampled, const int* sampled) {
    if (in_flight_.empty() || in_flight_.front().step != step) throw Failure{SCHEDULER_ERROR, "complete() must get the oldest plan in flight"};
    const Plan plan = std::move(in_flight_.front());
    in_flight_.pop_front();
    int wanted = 0;
    for (const PlanRow& row : plan.rows) wanted += row.sample;
    if (wanted != n_sampled) throw Failure{BAD_ARGUMENT, "the plan sampled " + std::to_string(wanted) + " tokens, " + std::to_string(n_sampled) + " were given"};
    const SchedulerConfig& c = config_;
    int index = -1;
    for (const PlanRow& row : plan.rows) {
        if (!row.sample) continue;
        ++index;
        auto found = running_.find(row.key);
        if (found == running_.end()) continue;  // cancelled, or ended by an end-of-sequence token, while this row was in flight
        Sequence& s = found->second;
        const int token = sampled[index];
        const bool is_eos = std::find(c.eos_token_ids.begin(), c.eos_token_ids.end(), token) != c.eos_token_ids.end();
        if (is_eos && !s.request.ignore_eos) {
            finish(row.key, "stop");
            continue;
        }
        ++s.generated;
        events_.push_back(Event{row.key, EVENT_TOKEN, token, ""});
        if (s.generated >= s.request.max_tokens || (int)s.request.prompt.size() + s.generated >= c.max_seq_len) {
            finish(row.key, "length");
        } else if (s.feed == Sequence::PLACE && s.feed_step == plan.step && s.feed_index == index) {
            s.feed = Sequence::TOKEN;  // no later plan has taken it from the device
            s.feed_token = token;
        }
    }
}

void Scheduler::fail(int step, const std::string& reason) {
    auto found = std::find_if(in_flight_.begin(), in_flight_.end(), [step](const Plan& p) { return p.step == step; });
    if (found == in_flight_.end()) throw Failure{SCHEDULER_ERROR, "fail() must get a plan in flight"};
    const Plan plan = std::move(*found);
    in_flight_.erase(found);
    for (const PlanRow& row : plan.rows) {
        if (!running_.count(row.key)) continue;
        drop(row.key);
        events_.push_back(Event{row.key, EVENT_FAILED, 0, reason});
    }
}

bool Scheduler::cancel(int64_t key) {
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
        if (it->key == key) {
            waiting_.erase(it);
            events_.push_back(Event{key, EVENT_FINISHED, 0, "cancelled"});
            return true;
        }
    if (!running_.count(key)) return false;
    finish(key, "cancelled");
    return true;
}

std::vector<Event> Scheduler::take_events() {
    std::vector<Event> events;
    events.swap(events_);
    return events;
}

std::vector<int64_t> Scheduler::take_released() {
    std::vector<int64_t> released;
    released.swap(released_);
    return released;
}

}  // namespace hb
