#include "scheduler.h"

#include <algorithm>

namespace cellm {

Scheduler::Scheduler(SchedulerConfig cfg, CacheManager* cache) : cfg_(cfg), cache_(cache) {
    if (cfg_.max_batch_tokens <= 0 || cfg_.prefill_chunk <= 0)
        throw SchedulerError("scheduler: token budget and portion size must be positive");
}

const Request& Scheduler::request(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw SchedulerError("scheduler: unknown request " + std::to_string(id));
    return it->second;
}

void Scheduler::add_request(int64_t id, const int32_t* tokens, int n, int max_new) {
    if (requests_.count(id)) throw SchedulerError("scheduler: request " + std::to_string(id) + " exists already");
    if (n <= 0) throw SchedulerError("scheduler: a request needs at least one prompt token");
    if (max_new < 1) throw SchedulerError("scheduler: a request must ask for at least one new token");
    const int total = n + max_new;
    if (total > cfg_.max_positions)
        throw SchedulerError("scheduler: prompt of " + std::to_string(n) + " tokens plus " + std::to_string(max_new) +
                             " new ones exceeds the model's " + std::to_string(cfg_.max_positions) + " positions");
    const int portion = std::min(cfg_.prefill_chunk, cfg_.max_batch_tokens);
    for (int g = 0; g < cache_->num_groups(); ++g) {
        const int need = cache_->pages_for(g, total, portion);
        if (need > cache_->group(g).num_pages)
            throw SchedulerError("scheduler: request " + std::to_string(id) + " needs " + std::to_string(need) +
                                 " pages of cache group " + std::to_string(g) + " for " + std::to_string(total) +
                                 " tokens, the pool has " + std::to_string(cache_->group(g).num_pages));
    }
    Request r;
    r.id = id;
    r.tokens.assign(tokens, tokens + n);
    r.prompt_len = n;
    r.max_new = max_new;
    requests_.emplace(id, std::move(r));
    waiting_.push_back(id);
}

int64_t Scheduler::newest_running() const {
    int64_t best = -1;
    uint64_t seq = 0;
    for (int64_t id : running_) {
        const Request& r = requests_.at(id);
        if (best < 0 || r.admit_seq > seq) { best = id; seq = r.admit_seq; }
    }
    return best;
}

void Scheduler::preempt(int64_t id, StepPlan& plan) {
    Request& r = requests_.at(id);
    cache_->release(id);
    r.computed = 0;
    r.state = RequestState::Waiting;
    r.preemptions++;
    preemptions_++;
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.push_front(id);
    plan.entries.erase(std::remove_if(plan.entries.begin(), plan.entries.end(),
                                      [id](const StepEntry& e) { return e.id == id; }),
                       plan.entries.end());
    plan.admitted.erase(std::remove_if(plan.admitted.begin(), plan.admitted.end(),
                                       [id](const std::pair<int64_t, int>& a) { return a.first == id; }),
                        plan.admitted.end());
    plan.preempted.push_back(id);
}

void Scheduler::finish(Request& r, const char* reason) {
    if (r.state == RequestState::Prefill || r.state == RequestState::Decoding) {
        cache_->release(r.id);
        running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    } else if (r.state == RequestState::Waiting) {
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r.id), waiting_.end());
    }
    r.state = RequestState::Finished;
    r.finish_reason = reason;
}

const StepPlan& Scheduler::schedule() {
    StepPlan& plan = plan_;
    plan = StepPlan{};
    for (int attempt = 0; attempt < 1 + (int)requests_.size(); ++attempt) {
        int budget = cfg_.max_batch_tokens;
        // 1. one token for each decoding request, in rotation order. While prompts are
        //    under way or waiting for a free slot, a quarter of the budget (at least one
        //    token) is kept for them, or decoders alone could fill every step for ever.
        std::vector<int64_t> decoders;
        bool prompt_work = !waiting_.empty() && cache_->free_slots() > 0;
        for (int64_t id : running_) {
            if (requests_.at(id).state == RequestState::Decoding) decoders.push_back(id);
            else prompt_work = true;
        }
        const int kept = (prompt_work && budget > 1) ? std::max(1, budget / 4) : 0;
        std::vector<int64_t> taken;
        for (int64_t id : decoders) {
            if (budget <= kept) break;
            if (!cache_->has(id)) continue;  // preempted a moment ago
            Request& r = requests_.at(id);
            if (r.state != RequestState::Decoding) continue;
            bool ok = cache_->reserve(id, r.computed + 1);
            while (!ok) {
                const int64_t victim = newest_running();
                if (victim == id && running_.size() == 1) {
                    // add_request checked that the request fits alone, so this cannot happen
                    // unless the pool was sized below what it promised.
                    finish(r, "out_of_pages");
                    break;
                }
                preempt(victim, plan);
                if (victim == id) break;
                ok = cache_->reserve(id, r.computed + 1);
            }
            if (!ok) continue;
            plan.entries.push_back({id, r.computed, 1, 1});
            taken.push_back(id);
            --budget;
        }
        // those served go to the back of the rotation (crates/cellm-scheduler/src/rr.rs:35-39)
        for (int64_t id : taken) {
            auto it = std::find(running_.begin(), running_.end(), id);
            if (it != running_.end()) { running_.erase(it); running_.push_back(id); }
        }
        // 2. portions of prompts that are under way
        std::vector<int64_t> prefilling;
        for (int64_t id : running_)
            if (requests_.at(id).state == RequestState::Prefill) prefilling.push_back(id);
        for (int64_t id : prefilling) {
            if (budget == 0) break;
            Request& r = requests_.at(id);
            int n = std::min({(int)r.tokens.size() - r.computed, cfg_.prefill_chunk, budget});
            while (n > 0 && !cache_->reserve(id, r.computed + n)) {
                // shrink to the next page edge below
                const int edge = ((r.computed + n - 1) / cache_->page_size()) * cache_->page_size();
                n = edge - r.computed;
            }
            if (n <= 0) continue;
            plan.entries.push_back({id, r.computed, n, r.computed + n == (int)r.tokens.size() ? 1 : 0});
            budget -= n;
        }
        // 3. admission in arrival order; none in a step that had to preempt, or the
        //    pages just freed would go straight back to the request they were taken from
        while (budget > 0 && !waiting_.empty() && plan.preempted.empty()) {
            const int64_t id = waiting_.front();
            Request& r = requests_.at(id);
            const int slot = cache_->add_request(id);
            if (slot < 0) break;
            // Admit only if the pool could hold all the tokens the request has now;
            // otherwise it would start, starve a decoding request of pages and be
            // preempted again at once. A windowed group holds only its window plus one
            // portion of them at a time (the measure add_request accepted the request by).
            int n = std::min({(int)r.tokens.size(), cfg_.prefill_chunk, budget});
            const int portion = std::min(cfg_.prefill_chunk, cfg_.max_batch_tokens);
            if (!cache_->can_hold(id, (int)r.tokens.size(), portion) || !cache_->reserve(id, n)) { cache_->release(id); break; }
            waiting_.pop_front();
            running_.push_back(id);
            r.state = RequestState::Prefill;
            r.computed = 0;
            r.admit_seq = ++admit_counter_;
            plan.admitted.push_back({id, slot});
            plan.entries.push_back({id, 0, n, n == (int)r.tokens.size() ? 1 : 0});
            budget -= n;
        }
        if (!plan.entries.empty() || running_.empty()) break;
        // Nothing can move although requests are running: they hold each other's pages.
        const int64_t victim = newest_running();
        if (running_.size() == 1) { finish(requests_.at(victim), "out_of_pages"); break; }
        preempt(victim, plan);
    }
    if (!plan.entries.empty()) {
        ++steps_;
        for (const auto& e : plan.entries) tokens_scheduled_ += (uint64_t)e.count;
    }
    return plan;
}

void Scheduler::step_done(const StepPlan& plan) {
    for (const auto& e : plan.entries) {
        Request& r = requests_.at(e.id);
        r.computed = e.start + e.count;
        cache_->commit(e.id, r.computed);
        if (r.state == RequestState::Prefill && r.computed == (int)r.tokens.size()) r.state = RequestState::Decoding;
    }
}

bool Scheduler::append_token(int64_t id, int32_t token, bool stop) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw SchedulerError("scheduler: unknown request " + std::to_string(id));
    Request& r = it->second;
    if (r.state != RequestState::Decoding)
        throw SchedulerError("scheduler: request " + std::to_string(id) + " is not decoding");
    if (r.computed != (int)r.tokens.size())
        throw SchedulerError("scheduler: request " + std::to_string(id) + " got a token before its last one ran");
    r.tokens.push_back(token);
    r.generated++;
    if (stop) { finish(r, "stop"); return true; }
    if (r.generated >= r.max_new) { finish(r, "length"); return true; }
    return false;
}

bool Scheduler::resolve_token(int64_t id, int index, int32_t token, bool stop) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return true;           // cancelled and forgotten meanwhile
    Request& r = it->second;
    if (index < r.prompt_len || index >= (int)r.tokens.size() || r.tokens[index] != PENDING_TOKEN)
        throw SchedulerError("scheduler: request " + std::to_string(id) + " has no pending token at " + std::to_string(index));
    r.tokens[index] = token;
    if (stop) {
        // the request ends here; a token appended after this one came from a step that ran on it
        if (r.state != RequestState::Finished) finish(r, "stop");
        else r.finish_reason = "stop";
        r.tokens.resize((size_t)index + 1);
        r.generated = index + 1 - r.prompt_len;
        return true;
    }
    return r.state == RequestState::Finished;
}

void Scheduler::cancel(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw SchedulerError("scheduler: unknown request " + std::to_string(id));
    if (it->second.state != RequestState::Finished) finish(it->second, "cancelled");
}

void Scheduler::forget(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return;
    if (it->second.state != RequestState::Finished)
        throw SchedulerError("scheduler: request " + std::to_string(id) + " is still live");
    requests_.erase(it);
}

}  // namespace cellm
