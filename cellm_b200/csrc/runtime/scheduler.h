// Continuous scheduler above the step function.
//
// The reference's engine prefills a whole prompt synchronously on submission
// and then rotates sessions one token at a time
// (crates/cellm-sdk/src/lib.rs:261-393, crates/cellm-scheduler/src/rr.rs:8-41,
// states in crates/cellm-scheduler/src/session.rs:5-109). Here every step is
// one batch under a token budget: each decoding request contributes one token,
// prompts are cut into portions that fill what is left of the budget, and
// waiting requests are admitted in arrival order while a state slot and pages
// are free. Rotation decides who goes first when the budget cannot take all.
//
// When pages run out: a decoding request that needs a page nobody can give
// makes the scheduler preempt the most recently admitted running request: its
// pages and slot are freed and it goes back to the head of the waiting queue,
// to be recomputed from its prompt plus the tokens it has generated so far.
// A request that could not fit even alone in an empty pool is refused when it
// is added.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <string>
#include <vector>

#include "cache_manager.h"

namespace cellm {

struct SchedulerError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

enum class RequestState : int { Waiting = 0, Prefill = 1, Decoding = 2, Finished = 3 };

struct Request {
    int64_t id = 0;
    std::vector<int32_t> tokens;  // prompt followed by generated tokens
    int prompt_len = 0;
    int max_new = 0;
    int computed = 0;             // tokens whose state is in the cache
    int generated = 0;
    int preemptions = 0;
    uint64_t admit_seq = 0;
    RequestState state = RequestState::Waiting;
    std::string finish_reason;
};

struct StepEntry {
    int64_t id;
    int start;        // position of the first token of this portion
    int count;        // tokens of the request that run in this step
    int wants_logits; // 1 when the portion ends at the request's last known token
};

struct StepPlan {
    std::vector<StepEntry> entries;
    std::vector<int64_t> preempted;                    // requests sent back to the waiting queue
    std::vector<std::pair<int64_t, int>> admitted;     // (request, state slot) newly admitted: slot must be zeroed
};

struct SchedulerConfig {
    int max_batch_tokens = 2048;
    int prefill_chunk = 2048;
    int max_positions = 1 << 30;
};

class Scheduler {
public:
    Scheduler(SchedulerConfig cfg, CacheManager* cache);

    void add_request(int64_t id, const int32_t* tokens, int n, int max_new);
    // Plans the next step. The plan is also kept as last_plan() until the next call, so that the
    // calls that follow a step (index arrays, step_done, sampled tokens) refer to this scheduler's own plan.
    const StepPlan& schedule();
    const StepPlan& last_plan() const { return plan_; }
    // To be called after the step of `plan` has run: marks the tokens as cached.
    void step_done(const StepPlan& plan);
    // Appends a sampled token; returns true when the request is finished
    // (max_new reached or `stop` set), in which case its pages and slot are freed.
    bool append_token(int64_t id, int32_t token, bool stop);
    // A token may be appended as PENDING_TOKEN while the step that forms it still runs (the engine launches the
    // next step before it has read this one's tokens; the kernels take the value from the device). resolve_token
    // gives the value of the pending token at `index` of the request's tokens later. With `stop` the request ends
    // at that token: whatever was appended after it is dropped. Returns true when the request is finished or gone.
    static constexpr int32_t PENDING_TOKEN = -1;
    bool resolve_token(int64_t id, int index, int32_t token, bool stop);
    void cancel(int64_t id);
    void forget(int64_t id);  // drops a finished request's record

    const Request& request(int64_t id) const;
    const CacheManager& cache() const { return *cache_; }
    bool has(int64_t id) const { return requests_.count(id) != 0; }
    int num_waiting() const { return (int)waiting_.size(); }
    int num_running() const { return (int)running_.size(); }
    bool idle() const { return waiting_.empty() && running_.empty(); }
    uint64_t steps() const { return steps_; }
    uint64_t tokens_scheduled() const { return tokens_scheduled_; }
    uint64_t preemptions() const { return preemptions_; }

private:
    void preempt(int64_t id, StepPlan& plan);
    void finish(Request& r, const char* reason);
    int64_t newest_running() const;

    SchedulerConfig cfg_;
    CacheManager* cache_;
    StepPlan plan_;
    std::map<int64_t, Request> requests_;
    std::deque<int64_t> waiting_;
    std::deque<int64_t> running_;  // rotation order
    uint64_t admit_counter_ = 0, steps_ = 0, tokens_scheduled_ = 0, preemptions_ = 0;
};

}  // namespace cellm
