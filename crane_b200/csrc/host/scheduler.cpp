#include "scheduler.hpp"

#include <algorithm>

#define CRANE_HOST_API extern "C" __attribute__((visibility("default")))

namespace crane {

int Scheduler::add(int64_t id, const int32_t* prompt, int n, int max_new_tokens,
                   const int32_t* eos, int n_eos) {
    if (seqs_.count(id)) return -2;
    if (n <= 0 || n > cfg_.max_seq_len) {
        ++stats_.rejected;
        return -1;
    }
    Sequence s;
    s.id = id;
    s.tokens.assign(prompt, prompt + n);
    s.prompt_len = n;
    s.max_new_tokens = std::max(0, std::min(max_new_tokens, cfg_.max_seq_len - n));
    s.eos.assign(eos, eos + n_eos);
    ++stats_.requests;
    stats_.prompt_tokens += n;
    if (s.max_new_tokens == 0) {
        s.finish = FinishReason::Length;   // nothing may be generated: done at once
        ++stats_.finished;
        seqs_.emplace(id, std::move(s));
        return 1;
    }
    seqs_.emplace(id, std::move(s));
    waiting_.push_back(id);
    return 0;
}

const Sequence* Scheduler::find(int64_t id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? nullptr : &it->second;
}

void Scheduler::finish(Sequence& s, FinishReason why) {
    if (s.finish != FinishReason::None) return;
    if (s.running) {
        cache_->release(s.id);
        s.running = false;
        running_.erase(std::remove(running_.begin(), running_.end(), s.id), running_.end());
    } else {
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), s.id), waiting_.end());
    }
    if (s.unresolved > 0) {                           // tokens that nobody will read any more
        s.tokens.resize(s.tokens.size() - s.unresolved);
        s.unresolved = 0;
    }
    s.finish = why;
    ++stats_.finished;
}

// The largest portion <= want whose pages are free now.
int Scheduler::fit(const Sequence& s, int want) const {
    int lo = 0, hi = want;   // lo always fits (0 tokens need no page)
    while (lo < hi) {
        const int mid = (lo + hi + 1) / 2;
        bool ok = true;
        for (int g = 0; g < cache_->num_groups() && ok; ++g)
            ok = cache_->pages_needed(s.id, mid, g) <= cache_->free_pages(g);
        if (ok) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Takes the cache of the most recently admitted request away.  Returns its id.
static int64_t latest(const std::deque<int64_t>& running) { return running.back(); }

bool Scheduler::preempt_one(int64_t /*keep*/, std::vector<PlanEntry>& plan, int& budget) {
    if (running_.size() <= 1) return false;
    const int64_t victim = latest(running_);
    Sequence& v = seqs_[victim];
    cache_->release(victim);
    v.running = false;
    v.computed = 0;
    ++v.preemptions;
    ++stats_.preemptions;
    running_.pop_back();
    waiting_.push_front(victim);
    last_preempted_.push_back(victim);
    for (auto it = plan.begin(); it != plan.end(); ++it)
        if (it->id == victim) {
            budget += it->count;
            plan.erase(it);
            break;
        }
    return true;
}

std::vector<PlanEntry> Scheduler::schedule(std::vector<int32_t>& tokens) {
    std::vector<PlanEntry> plan;
    tokens.clear();
    last_preempted_.clear();
    last_failed_.clear();
    int budget = cfg_.max_batched_tokens;

    // pass 0: one token of every decoding request; pass 1: prompt portions of
    // the requests that already hold cache
    for (int pass = 0; pass < 2; ++pass) {
        const std::vector<int64_t> snapshot(running_.begin(), running_.end());
        for (int64_t id : snapshot) {
            Sequence& s = seqs_[id];
            if (!s.running) continue;                 // preempted a moment ago
            if (s.closing) continue;                  // waits for its last token only
            const int pend = s.pending();
            if (pend <= 0) continue;
            if ((pass == 0) != (pend == 1)) continue;
            if (budget <= 0) break;
            int n = std::min(std::min(pend, cfg_.chunk_size), budget);
            bool self = false;
            while (cache_->extend(id, n) != 0) {
                if (running_.size() > 1) {
                    const int64_t victim = latest(running_);
                    preempt_one(id, plan, budget);
                    if (victim == id) { self = true; break; }
                } else {
                    n = fit(s, n);
                    if (n <= 0) break;
                }
            }
            if (self) continue;
            if (n <= 0) {                             // alone, and not one more token fits
                finish(s, FinishReason::CacheTooSmall);
                last_failed_.push_back(id);
                continue;
            }
            plan.push_back({id, s.computed, n, s.computed + n == (int)s.tokens.size() ? 1 : 0});
            s.computed += n;
            budget -= n;
        }
    }
    // admission: FIFO, never by taking pages from a request that holds some
    while (!waiting_.empty() && (int)running_.size() < cfg_.max_running && budget > 0 &&
           cache_->free_slots() > 0) {
        const int64_t id = waiting_.front();
        Sequence& s = seqs_[id];
        if (s.closing) break;                         // only its last token is still to come
        int n = std::min(std::min(s.pending(), cfg_.chunk_size), budget);
        if (cache_->admit(id) < 0) break;
        if (cache_->extend(id, n) != 0) {
            if (!running_.empty()) {                  // wait until someone finishes
                cache_->release(id);
                break;
            }
            n = fit(s, n);                            // alone: take what the pool can hold
            if (n <= 0 || cache_->extend(id, n) != 0) {
                cache_->release(id);
                waiting_.pop_front();
                s.tokens.resize(s.tokens.size() - s.unresolved);
                s.unresolved = 0;
                s.finish = FinishReason::CacheTooSmall;
                ++stats_.finished;
                last_failed_.push_back(id);
                continue;
            }
        }
        waiting_.pop_front();
        running_.push_back(id);
        s.running = true;
        s.admit_stamp = ++stamp_;
        plan.push_back({id, s.computed, n, s.computed + n == (int)s.tokens.size() ? 1 : 0});
        s.computed += n;
        budget -= n;
    }
    for (const PlanEntry& e : plan) {
        const Sequence& s = seqs_[e.id];
        tokens.insert(tokens.end(), s.tokens.begin() + e.start, s.tokens.begin() + e.start + e.count);
        stats_.scheduled_tokens += e.count;
    }
    if (!plan.empty()) ++stats_.steps;
    return plan;
}

FinishReason Scheduler::on_token(int64_t id, int32_t token) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return FinishReason::None;
    Sequence& s = it->second;
    if (s.finish != FinishReason::None) return s.finish;
    s.tokens.push_back(token);
    ++stats_.generated_tokens;
    if (std::find(s.eos.begin(), s.eos.end(), token) != s.eos.end())
        finish(s, FinishReason::Stop);
    else if (s.generated() >= s.max_new_tokens || (int)s.tokens.size() >= cfg_.max_seq_len)
        finish(s, FinishReason::Length);
    return s.finish;
}

void Scheduler::expect_token(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end() || it->second.finish != FinishReason::None) return;
    Sequence& s = it->second;
    s.tokens.push_back(-1);
    ++s.unresolved;
    if (s.generated() >= s.max_new_tokens || (int)s.tokens.size() >= cfg_.max_seq_len) s.closing = true;
}

FinishReason Scheduler::resolve_token(int64_t id, int32_t token) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return FinishReason::None;
    Sequence& s = it->second;
    if (s.finish != FinishReason::None || s.unresolved <= 0) return s.finish;
    const int idx = (int)s.tokens.size() - s.unresolved;
    s.tokens[idx] = token;
    --s.unresolved;
    ++stats_.generated_tokens;
    const int gen = idx + 1 - s.prompt_len;
    const bool stop = std::find(s.eos.begin(), s.eos.end(), token) != s.eos.end();
    if (stop || gen >= s.max_new_tokens || idx + 1 >= cfg_.max_seq_len) {
        s.tokens.resize(idx + 1);                     // what was planned beyond it is void
        s.unresolved = 0;
        finish(s, stop ? FinishReason::Stop : FinishReason::Length);
    }
    return s.finish;
}

int Scheduler::cancel(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return -2;
    finish(it->second, FinishReason::Cancelled);
    return 0;
}

int Scheduler::drop(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return -2;
    if (it->second.finish == FinishReason::None) return -1;
    seqs_.erase(it);
    return 0;
}

}  // namespace crane

using crane::Scheduler;

CRANE_HOST_API void* crane_sched_create(void* cache, int max_running, int max_batched_tokens,
                                        int chunk_size, int max_seq_len) {
    if (!cache || max_running <= 0 || max_batched_tokens <= 0 || chunk_size <= 0 || max_seq_len <= 0)
        return nullptr;
    return new Scheduler((crane::CacheManager*)cache,
                         {max_running, max_batched_tokens, chunk_size, max_seq_len});
}
CRANE_HOST_API void crane_sched_destroy(void* s) { delete (Scheduler*)s; }
CRANE_HOST_API int crane_sched_add(void* s, int64_t id, const int32_t* prompt, int n, int max_new,
                                   const int32_t* eos, int n_eos) {
    return ((Scheduler*)s)->add(id, prompt, n, max_new, eos, n_eos);
}
// Returns the number of entries, or -1 if a caller's array is too small.
CRANE_HOST_API int crane_sched_schedule(void* s, int64_t* ids, int32_t* start, int32_t* count,
                                        int32_t* sample, int cap_entries, int32_t* tokens,
                                        int cap_tokens, int32_t* n_tokens) {
    std::vector<int32_t> toks;
    auto plan = ((Scheduler*)s)->schedule(toks);
    if ((int)plan.size() > cap_entries || (int)toks.size() > cap_tokens) return -1;
    for (size_t i = 0; i < plan.size(); ++i) {
        ids[i] = plan[i].id;
        start[i] = plan[i].start;
        count[i] = plan[i].count;
        sample[i] = plan[i].sample;
    }
    std::copy(toks.begin(), toks.end(), tokens);
    *n_tokens = (int)toks.size();
    return (int)plan.size();
}
CRANE_HOST_API int crane_sched_on_token(void* s, int64_t id, int32_t tok) {
    return (int)((Scheduler*)s)->on_token(id, tok);
}
// The tokens sampled for several entries at once; reasons[i] gets the finish reason.
CRANE_HOST_API void crane_sched_on_tokens(void* s, int n, const int64_t* ids, const int32_t* toks,
                                          int32_t* reasons) {
    for (int i = 0; i < n; ++i) reasons[i] = (int)((Scheduler*)s)->on_token(ids[i], toks[i]);
}
CRANE_HOST_API void crane_sched_expect_tokens(void* s, int n, const int64_t* ids) {
    for (int i = 0; i < n; ++i) ((Scheduler*)s)->expect_token(ids[i]);
}
CRANE_HOST_API void crane_sched_resolve_tokens(void* s, int n, const int64_t* ids, const int32_t* toks,
                                               int32_t* reasons) {
    for (int i = 0; i < n; ++i) reasons[i] = (int)((Scheduler*)s)->resolve_token(ids[i], toks[i]);
}
CRANE_HOST_API int crane_sched_cancel(void* s, int64_t id) { return ((Scheduler*)s)->cancel(id); }
CRANE_HOST_API int crane_sched_drop(void* s, int64_t id) { return ((Scheduler*)s)->drop(id); }
CRANE_HOST_API int crane_sched_has_work(void* s) { return ((Scheduler*)s)->has_work() ? 1 : 0; }
CRANE_HOST_API int crane_sched_num_waiting(void* s) { return ((Scheduler*)s)->num_waiting(); }
CRANE_HOST_API int crane_sched_num_running(void* s) { return ((Scheduler*)s)->num_running(); }
// state of one request: out[0]=finish reason, [1]=prompt_len, [2]=total tokens,
// [3]=computed, [4]=running, [5]=preemptions.  -2 unknown id.
CRANE_HOST_API int crane_sched_state(void* s, int64_t id, int32_t* out) {
    const crane::Sequence* q = ((Scheduler*)s)->find(id);
    if (!q) return -2;
    out[0] = (int)q->finish;
    out[1] = q->prompt_len;
    out[2] = (int)q->tokens.size();
    out[3] = q->computed;
    out[4] = q->running ? 1 : 0;
    out[5] = q->preemptions;
    return 0;
}
CRANE_HOST_API int crane_sched_tokens(void* s, int64_t id, int32_t* out, int cap) {
    const crane::Sequence* q = ((Scheduler*)s)->find(id);
    if (!q) return -2;
    const int n = std::min(cap, (int)q->tokens.size());
    std::copy(q->tokens.begin(), q->tokens.begin() + n, out);
    return (int)q->tokens.size();
}
CRANE_HOST_API void crane_sched_stats(void* s, int64_t* out) {
    const crane::Stats& t = ((Scheduler*)s)->stats();
    out[0] = t.steps; out[1] = t.requests; out[2] = t.finished; out[3] = t.prompt_tokens;
    out[4] = t.generated_tokens; out[5] = t.scheduled_tokens; out[6] = t.preemptions;
    out[7] = t.rejected;
}
CRANE_HOST_API int crane_sched_last_preempted(void* s, int64_t* out, int cap) {
    const auto& v = ((Scheduler*)s)->last_preempted();
    const int n = std::min(cap, (int)v.size());
    std::copy(v.begin(), v.begin() + n, out);
    return (int)v.size();
}
CRANE_HOST_API int crane_sched_last_failed(void* s, int64_t* out, int cap) {
    const auto& v = ((Scheduler*)s)->last_failed();
    const int n = std::min(cap, (int)v.size());
    std::copy(v.begin(), v.begin() + n, out);
    return (int)v.size();
}
