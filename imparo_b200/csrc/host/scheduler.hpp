// Continuous-batching decisions above the step function.  It counts tokens; the token
// values stay with the caller.
//
// Taken from the reference's engine loop (imparo-server/src/sched.rs:187-318): requests
// wait in arrival order; every decoding request gets one token per step; prompts enter in
// portions under a token budget (there one 512-token chunk per iteration, sched.rs:292-310;
// imparo-model/src/lib.rs:1000); a request joins the decoders with the token sampled from
// its last portion's logits (sched.rs:424-442), so N new tokens cost N-1 decode steps;
// max_tokens == 0 ends before any token (sched.rs:427-431); admission wants the prompt's
// pages plus one spare page per running row (sched.rs:340-346); a failed step abandons
// every request in it (sched.rs:652-660).
// Different on purpose: prompt portions and decode tokens share ONE step; several prompts
// may be in flight; and when pages run out the NEWEST running request is preempted — its
// pages and slot go back and it re-enters at the head of the queue with prompt plus
// generated tokens as its new prompt (the reference parks to a disk tier instead,
// sched.rs:662-808).  A request that cannot get pages even alone fails with
// "context exceeds pool".
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <vector>

#include "cache_manager.hpp"

namespace imparo {

struct PlanEntry {
    int64_t id;
    int start;      // position of the first token of this portion
    int count;      // tokens in this portion
    int want;       // 1: logits of the portion's last token are needed (a token will be sampled)
};

// How many one-token rows a step runs when n requests bring one token each: up to 8 the next power of two,
// above that the next multiple of 8.  The step function fills the difference with rows that belong to no
// request (they write to the cache's spare page and slot), so that the steps of a continuous batch, whose
// number of decoding requests changes by one every few steps, fall into few shapes and replay captured graphs.
inline int padded_rows(int n) {
    if (n <= 1) return n < 0 ? 0 : n;
    if (n <= 8) { int p = 1; while (p < n) p <<= 1; return p; }
    return (n + 7) / 8 * 8;
}

class Scheduler {
public:
    Scheduler(CacheManager* cm, int max_step_tokens, int max_running, int max_context);

    // true: the token budget counts the rows the step function will add beside the one-token requests
    // (padded_rows), so that a step with prompt portions holds exactly max_step_tokens rows whenever prompts
    // are left, whatever the number of decoding requests.
    void count_padded_rows(bool on) { count_padded_rows_ = on; }

    int64_t submit(int prompt_len, int max_new_tokens);
    // Decide the next step.  Entries: decode tokens first (admission order), then prompt
    // portions.  Empty when nothing can run.
    const std::vector<PlanEntry>& plan();
    // The planned step ran (ok) or failed.  ok: caches advance.  failed: every request in
    // the plan is abandoned and what it held goes back.
    void step_done(bool ok);
    // A token was sampled for a request that wanted logits.  Returns 1 when the request is
    // finished (eos, max_new_tokens or the context limit) and has been released.
    int on_token(int64_t id, bool is_eos);
    int abort(int64_t id);

    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int n_waiting() const { return (int)waiting_.size(); }
    int n_running() const { return (int)running_.size(); }
    // Drained by the caller: requests preempted / failed since the last call.
    std::vector<int64_t> take_preempted();
    std::vector<int64_t> take_failed();
    int64_t n_preemptions() const { return n_preemptions_; }
    int64_t n_steps() const { return n_steps_; }
    int known_tokens(int64_t id) const;
    int generated(int64_t id) const;

private:
    struct Req {
        int known = 0;        // prompt + generated tokens whose values the caller holds
        int generated = 0;
        int max_new = 0;
        int64_t order = 0;    // admission order (larger = newer)
    };
    bool preempt_newest(int64_t keep);
    void fail(int64_t id);

    CacheManager* cm_;
    int max_step_tokens_, max_running_, max_context_;
    int64_t next_id_ = 1, next_order_ = 1;
    std::map<int64_t, Req> reqs_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;          // admission order
    std::vector<PlanEntry> plan_;
    std::vector<int64_t> preempted_, failed_;
    int64_t n_preemptions_ = 0, n_steps_ = 0;
    bool count_padded_rows_ = false;
};

}  // namespace imparo
