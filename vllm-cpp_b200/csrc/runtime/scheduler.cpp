#include "scheduler.h"

#include <algorithm>
#include <stdexcept>

namespace vcb {

Scheduler::Scheduler(std::vector<GroupSpec> groups, int32_t max_num_seqs, int32_t max_step_tokens,
                     int32_t max_model_len)
    : cache_(std::move(groups), max_num_seqs),
      max_num_seqs_(max_num_seqs),
      max_step_tokens_(max_step_tokens),
      max_model_len_(max_model_len) {
    if (max_num_seqs < 1 || max_step_tokens < 1 || max_model_len < 1)
        throw std::invalid_argument("scheduler limits must be >= 1");
}

bool Scheduler::fits_empty_pool(int32_t total_len) const {
    for (int32_t g = 0; g < cache_.num_groups(); ++g)
        if (cache_.peak_pages(g, total_len, max_step_tokens_) > cache_.group(g).num_pages) return false;
    return true;
}

int64_t Scheduler::submit(std::vector<int32_t> prompt, int32_t max_new_tokens, SamplingParams sampling,
                          std::vector<int32_t> stop_ids) {
    if (prompt.empty()) throw std::invalid_argument("submit: the prompt is empty");
    if (max_new_tokens < 1) throw std::invalid_argument("submit: max_new_tokens must be >= 1");
    const int64_t total = (int64_t)prompt.size() + max_new_tokens;
    if (total > max_model_len_)
        throw std::invalid_argument("submit: prompt (" + std::to_string(prompt.size()) + ") + max_new_tokens (" +
                                    std::to_string(max_new_tokens) + ") exceeds max_model_len " +
                                    std::to_string(max_model_len_));
    if (!fits_empty_pool((int32_t)total))
        throw std::invalid_argument("submit: a request of " + std::to_string(total) +
                                    " tokens does not fit the cache pool even when it is empty");
    Request r;
    r.id = next_id_++;
    r.prompt = std::move(prompt);
    r.max_new_tokens = max_new_tokens;
    r.sampling = sampling;
    r.stop_ids = std::move(stop_ids);
    const int64_t id = r.id;
    requests_.emplace(id, std::move(r));
    waiting_.push_back(id);
    return id;
}

const Request& Scheduler::request(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw std::invalid_argument("unknown request " + std::to_string(id));
    return it->second;
}

int32_t Scheduler::num_finished() const {
    int32_t n = 0;
    for (const auto& kv : requests_) n += kv.second.state == RequestState::FINISHED;
    return n;
}

void Scheduler::preempt(int64_t id, SchedulerOutput& out) {
    Request& r = requests_.at(id);
    cache_.close(id);
    stats_.preemptions++;
    stats_.recomputed_tokens += r.num_computed;
    r.num_computed = 0;
    r.slot = -1;
    r.state = RequestState::PREEMPTED;
    r.preempt_count++;
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.push_front(id);
    out.preempted.push_back(id);
}

void Scheduler::finish(Request& r, const std::string& reason) {
    if (cache_.is_open(r.id)) cache_.close(r.id);
    r.state = RequestState::FINISHED;
    r.finish_reason = reason;
    r.slot = -1;
    running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r.id), waiting_.end());
}

bool Scheduler::room_to_admit(const Request& r, int32_t first_portion) const {
    // like the reference's can_allocate (src/scheduler.cpp:67-72): the pages of the whole current
    // sequence must be free now, although only the first portion's are taken
    for (int32_t g = 0; g < cache_.num_groups(); ++g) {
        const int32_t want = std::max(cache_.peak_pages(g, r.seq_len(), max_step_tokens_),
                                      cache_.pages_missing(-1, g, first_portion));
        if (want > cache_.free_pages(g)) return false;
    }
    return true;
}

SchedulerOutput Scheduler::schedule() {
    if (awaiting_update_) throw std::logic_error("schedule() called again before update()");
    SchedulerOutput out;
    int32_t budget = max_step_tokens_;

    // 1. requests already running, oldest first: one decoded token each, or the next portion of a prompt
    for (size_t i = 0; i < running_.size() && budget > 0;) {
        Request& r = requests_.at(running_[i]);
        const int32_t remaining = r.seq_len() - r.num_computed;
        const int32_t n = std::min(remaining, budget);
        bool self_preempted = false;
        while (!cache_.reserve(r.id, r.num_computed + n)) {
            const int64_t victim = running_.back();
            preempt(victim, out);
            if (victim == r.id) {
                self_preempted = true;
                break;
            }
        }
        if (self_preempted) break;  // it was the last of the running list
        ScheduledEntry e;
        e.request = r.id;
        e.slot = r.slot;
        e.start_pos = r.num_computed;
        e.tokens.reserve(n);
        for (int32_t k = 0; k < n; ++k) e.tokens.push_back(r.token_at(r.num_computed + k));
        e.sample = (r.num_computed + n == r.seq_len());
        e.gen_step = (int32_t)r.generated.size();
        // a decode entry feeds exactly one token, and that token was generated
        e.is_prompt = !(remaining == 1 && r.num_computed >= (int32_t)r.prompt.size());
        if (e.is_prompt) out.num_prompt_tokens += n; else out.num_generation_tokens += n;
        budget -= n;
        out.entries.push_back(std::move(e));
        ++i;
    }

    // 2. newcomers, first come first served; never in a step that had to preempt, never by preempting
    while (out.preempted.empty() && !waiting_.empty() && (int32_t)running_.size() < max_num_seqs_ && budget > 0) {
        Request& r = requests_.at(waiting_.front());
        const int32_t n = std::min(r.seq_len(), budget);
        if (!room_to_admit(r, n)) break;
        const int32_t slot = cache_.open(r.id);
        if (slot < 0) break;
        if (!cache_.reserve(r.id, n)) {
            cache_.close(r.id);
            break;
        }
        waiting_.pop_front();
        r.slot = slot;
        r.state = RequestState::RUNNING;
        r.num_computed = 0;
        running_.push_back(r.id);
        ScheduledEntry e;
        e.request = r.id;
        e.slot = slot;
        e.start_pos = 0;
        e.tokens.reserve(n);
        for (int32_t k = 0; k < n; ++k) e.tokens.push_back(r.token_at(k));
        e.sample = (n == r.seq_len());
        e.gen_step = (int32_t)r.generated.size();
        e.is_prompt = true;
        out.num_prompt_tokens += n;
        budget -= n;
        out.entries.push_back(std::move(e));
    }

    last_entries_ = out.entries;
    awaiting_update_ = !out.entries.empty();
    if (!out.entries.empty()) stats_.steps++;
    stats_.prompt_tokens += out.num_prompt_tokens;
    return out;
}

std::vector<int64_t> Scheduler::update(const std::vector<int32_t>& sampled) {
    if (!awaiting_update_) throw std::logic_error("update() without a scheduled step");
    size_t want = 0;
    for (const auto& e : last_entries_) want += e.sample;
    if (sampled.size() != want)
        throw std::invalid_argument("update: " + std::to_string(sampled.size()) + " tokens given, " +
                                    std::to_string(want) + " entries asked for one");
    std::vector<int64_t> finished;
    size_t k = 0;
    for (const auto& e : last_entries_) {
        auto it = requests_.find(e.request);
        const bool alive = it != requests_.end() && it->second.state == RequestState::RUNNING;
        const int32_t tok = e.sample ? sampled[k++] : -1;
        if (!alive) continue;  // aborted between schedule() and update()
        Request& r = it->second;
        r.num_computed += (int32_t)e.tokens.size();
        cache_.commit(r.id, r.num_computed);
        if (!e.sample) continue;
        r.generated.push_back(tok);
        stats_.generated_tokens++;
        const bool stop = std::find(r.stop_ids.begin(), r.stop_ids.end(), tok) != r.stop_ids.end();
        if (stop) finish(r, "stop");
        else if ((int32_t)r.generated.size() >= r.max_new_tokens || r.seq_len() >= max_model_len_) finish(r, "length");
        if (r.state == RequestState::FINISHED) finished.push_back(r.id);
    }
    last_entries_.clear();
    awaiting_update_ = false;
    return finished;
}

void Scheduler::abort(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return;
    if (it->second.state != RequestState::FINISHED) finish(it->second, "abort");
}

void Scheduler::forget(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return;
    if (it->second.state != RequestState::FINISHED) throw std::logic_error("forget() of an unfinished request");
    requests_.erase(it);
}

}  // namespace vcb
