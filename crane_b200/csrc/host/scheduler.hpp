// Continuous-batching scheduler: admits requests, cuts prompts into portions
// under a token budget, lets every admitted request decode one token per step,
// finishes requests and gives their pages back, and decides what happens when
// pages run out.
//
// Kept from the reference (crane-serve/src/engine/scheduler.rs:23-97,
// sequence.rs:62-116, mod.rs:610-651): FIFO queues `waiting` and `running`,
// at most `max_running` requests hold cache, a request stops after
// `max_new_tokens` generated tokens ("length") or on a token of its EOS set
// ("stop"), prompts longer than the sequence limit are refused and
// `max_new_tokens` is clamped to what the limit leaves.
// Changed: the reference prefills one whole prompt per step and never mixes it
// with decoding; here a step holds one token of every decoding request first
// and fills the rest of the budget with prompt portions.  When pages run out
// the reference drops the longest request's cache and truncates it to its
// prompt (mod.rs:533-590); here the most recently admitted request is
// preempted, keeps prompt and generated tokens, goes to the FRONT of `waiting`
// and is recomputed, so its output continues where it stopped.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.hpp"

namespace crane {

struct SchedulerConfig {
    int max_running;          // requests that may hold cache at once
    int max_batched_tokens;   // token budget of one step
    int chunk_size;           // longest prompt portion of one request in one step
    int max_seq_len;          // prompt + generated may not exceed this
};

enum class FinishReason : int { None = 0, Stop = 1, Length = 2, Cancelled = 3, CacheTooSmall = 4 };

struct Sequence {
    int64_t id = 0;
    std::vector<int32_t> tokens;     // prompt ++ generated
    int prompt_len = 0;
    int max_new_tokens = 0;
    std::vector<int32_t> eos;
    int computed = 0;                // tokens whose keys/values are in the cache
    bool running = false;            // holds a slot and pages
    FinishReason finish = FinishReason::None;
    int preemptions = 0;
    int64_t admit_stamp = 0;
    int unresolved = 0;              // placeholders (-1) at the end of `tokens`: sampled, not yet known
    bool closing = false;            // its last allowed token is sampled but not yet known: plan nothing more

    int generated() const { return (int)tokens.size() - prompt_len; }
    int pending() const { return (int)tokens.size() - computed; }
};

struct PlanEntry {
    int64_t id;
    int start;      // position of the first token of the portion
    int count;      // tokens in the portion
    int sample;     // 1: the portion ends at the request's last known token
};

struct Stats {
    int64_t steps = 0, requests = 0, finished = 0, prompt_tokens = 0, generated_tokens = 0,
            scheduled_tokens = 0, preemptions = 0, rejected = 0;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, const SchedulerConfig& cfg) : cache_(cache), cfg_(cfg) {}

    // 0: queued.  -1: prompt empty or longer than the limit (refused).  -2: id in use.
    int add(int64_t id, const int32_t* prompt, int n, int max_new_tokens, const int32_t* eos,
            int n_eos);
    // Builds the next step.  Returns the entries; `tokens` gets their token ids, flat.
    std::vector<PlanEntry> schedule(std::vector<int32_t>& tokens);
    // The token sampled for an entry whose `sample` was 1.  Returns the finish
    // reason (None: goes on).  A finished request has given its pages back.
    FinishReason on_token(int64_t id, int32_t token);
    // For engines that plan step N + 1 before the tokens sampled in step N have
    // come back from the device: expect_token() puts a placeholder (-1) where the
    // token will go, so that the request can be planned again (its next input is
    // then read on the device from the sampler's output); resolve_token() fills the
    // oldest placeholder in and applies the stop rules.  A request whose
    // placeholder is its last token by count is not planned again.  If the
    // resolved token stops the request, later placeholders are dropped.
    void expect_token(int64_t id);
    FinishReason resolve_token(int64_t id, int32_t token);
    int cancel(int64_t id);
    // Forget a finished request (its tokens stay readable until then).
    int drop(int64_t id);

    const Sequence* find(int64_t id) const;
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int num_waiting() const { return (int)waiting_.size(); }
    int num_running() const { return (int)running_.size(); }
    const Stats& stats() const { return stats_; }
    // ids preempted or finished for lack of cache by the last schedule() call
    const std::vector<int64_t>& last_preempted() const { return last_preempted_; }
    const std::vector<int64_t>& last_failed() const { return last_failed_; }

private:
    void finish(Sequence& s, FinishReason why);
    bool preempt_one(int64_t keep, std::vector<PlanEntry>& plan, int& budget);
    int fit(const Sequence& s, int want) const;

    CacheManager* cache_;
    SchedulerConfig cfg_;
    std::unordered_map<int64_t, Sequence> seqs_;
    std::deque<int64_t> waiting_;
    std::deque<int64_t> running_;   // in order of admission
    Stats stats_;
    int64_t stamp_ = 0;
    std::vector<int64_t> last_preempted_, last_failed_;
};

}  // namespace crane
