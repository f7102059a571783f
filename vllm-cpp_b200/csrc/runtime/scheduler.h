// Continuous-batching scheduler above the model step.
//
// Same job and request states as the reference's Scheduler (src/scheduler.h:28-107,
// src/request.h:9-55): FIFO admission, a running set, one decoded token per running
// request and step, finish on a stop token or on max_new_tokens.  What differs:
//  * a step has a token budget; prompts are fed in portions that fit what the
//    budget leaves after the decoding requests (the reference always feeds a prompt
//    whole, src/paged_engine.cpp:318, and bounds the sum of sequence lengths instead,
//    src/scheduler.cpp:221-235);
//  * pages are reserved portion by portion, not for the whole prompt at admission
//    (src/scheduler.cpp:74-85);
//  * when a running request cannot get its next page, the youngest running request
//    is preempted by *recompute*: its pages and slot go back, it returns to the head
//    of the waiting queue and later feeds prompt + generated tokens again.  (The
//    reference preempts to admit newcomers and restores from pages it has already
//    freed, src/scheduler.cpp:87-153, 194-218.)  Nothing is preempted to admit.
//  * resources are given back in the call that finishes a request, not in the next
//    schedule() (src/scheduler.cpp:245-264).
// Single-threaded by contract; the scheduler owns the CacheManager.
#pragma once
#include <cstdint>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.h"

namespace vcb {

enum class RequestState { WAITING, RUNNING, FINISHED, PREEMPTED };

struct SamplingParams {
    float temperature = 0.7f;     // the reference's TEMPERATURE (src/config.h:97); <= 0 is greedy
    float top_p = 0.8f;           // TOP_P (src/config.h:98)
    float repeat_penalty = 1.1f;  // REPEAT_PENALTY (src/config.h:99)
    uint64_t seed = 0;
};

struct Request {
    int64_t id = -1;
    std::vector<int32_t> prompt;
    std::vector<int32_t> generated;
    RequestState state = RequestState::WAITING;
    int32_t max_new_tokens = 2048;  // MAX_NEW_TOKENS (src/config.h:100)
    SamplingParams sampling;
    std::vector<int32_t> stop_ids;
    int32_t num_computed = 0;  // tokens of prompt + generated whose cache entries exist
    int32_t slot = -1;
    int32_t preempt_count = 0;
    std::string finish_reason;  // "stop", "length", "abort"

    int32_t seq_len() const { return (int32_t)(prompt.size() + generated.size()); }
    int32_t token_at(int32_t i) const {
        return i < (int32_t)prompt.size() ? prompt[i] : generated[i - (int32_t)prompt.size()];
    }
};

// One request's share of a step: tokens [start_pos, start_pos + tokens.size()) of its sequence.
struct ScheduledEntry {
    int64_t request = -1;
    int32_t slot = -1;
    int32_t start_pos = 0;
    std::vector<int32_t> tokens;
    bool sample = false;    // the portion ends the known sequence: its last logits choose the next token
    int32_t gen_step = 0;   // index of the token to be sampled among the generated ones
    bool is_prompt = false; // the portion holds prompt (or recomputed) tokens rather than one decoded token
};

struct SchedulerOutput {
    std::vector<ScheduledEntry> entries;
    std::vector<int64_t> preempted;
    int32_t num_prompt_tokens = 0;
    int32_t num_generation_tokens = 0;
};

struct SchedulerStats {
    int64_t steps = 0, preemptions = 0, recomputed_tokens = 0, prompt_tokens = 0, generated_tokens = 0;
};

class Scheduler {
public:
    Scheduler(std::vector<GroupSpec> groups, int32_t max_num_seqs, int32_t max_step_tokens, int32_t max_model_len);

    // Queues a request; throws std::invalid_argument when it could never run (empty prompt, longer than
    // max_model_len, or too large for an empty pool).
    int64_t submit(std::vector<int32_t> prompt, int32_t max_new_tokens, SamplingParams sampling,
                   std::vector<int32_t> stop_ids);
    // Chooses the tokens of the next step and reserves their pages.
    SchedulerOutput schedule();
    // Takes the sampled tokens of the entries that asked for one (same order as the entries with
    // sample == true).  Returns the ids of requests that finished.
    std::vector<int64_t> update(const std::vector<int32_t>& sampled);
    // Finishes a request now (reason "abort"), whatever its state.
    void abort(int64_t request);
    // Drops a finished request's record.
    void forget(int64_t request);

    bool has_unfinished() const { return !waiting_.empty() || !running_.empty(); }
    const Request& request(int64_t id) const;
    bool knows(int64_t id) const { return requests_.count(id) != 0; }
    int32_t num_waiting() const { return (int32_t)waiting_.size(); }
    int32_t num_running() const { return (int32_t)running_.size(); }
    int32_t num_finished() const;
    const SchedulerStats& stats() const { return stats_; }
    CacheManager& cache() { return cache_; }
    const CacheManager& cache() const { return cache_; }
    int32_t max_step_tokens() const { return max_step_tokens_; }
    int32_t max_num_seqs() const { return max_num_seqs_; }
    int32_t max_model_len() const { return max_model_len_; }

private:
    void preempt(int64_t id, SchedulerOutput& out);
    void finish(Request& r, const std::string& reason);
    bool fits_empty_pool(int32_t total_len) const;
    bool room_to_admit(const Request& r, int32_t first_portion) const;

    CacheManager cache_;
    int32_t max_num_seqs_, max_step_tokens_, max_model_len_;
    int64_t next_id_ = 0;
    std::unordered_map<int64_t, Request> requests_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;  // admission order: back() is the youngest
    std::vector<ScheduledEntry> last_entries_;
    bool awaiting_update_ = false;
    SchedulerStats stats_;
};

}  // namespace vcb
