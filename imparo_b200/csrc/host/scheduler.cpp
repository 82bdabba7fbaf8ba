#include "scheduler.hpp"

#include <algorithm>
#include <set>

namespace imparo {

Scheduler::Scheduler(CacheManager* cm, int max_step_tokens, int max_running, int max_context)
    : cm_(cm), max_step_tokens_(std::max(1, max_step_tokens)), max_running_(std::max(1, max_running)),
      max_context_(max_context) {}

int64_t Scheduler::submit(int prompt_len, int max_new_tokens) {
    if (prompt_len < 1 || max_new_tokens < 1 || prompt_len > max_context_) return -1;
    const int64_t id = next_id_++;
    Req r;
    r.known = prompt_len;
    r.max_new = max_new_tokens;
    reqs_[id] = r;
    waiting_.push_back(id);
    return id;
}

void Scheduler::fail(int64_t id) {
    cm_->release(id);
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    reqs_.erase(id);
    failed_.push_back(id);
}

bool Scheduler::preempt_newest(int64_t /*keep*/) {
    if (running_.size() < 2) return false;
    int64_t newest = -1, best = -1;
    for (int64_t id : running_)
        if (reqs_[id].order > best) { best = reqs_[id].order; newest = id; }
    cm_->release(newest);
    running_.erase(std::remove(running_.begin(), running_.end(), newest), running_.end());
    waiting_.push_front(newest);          // it re-enters first, its prompt = all it has so far
    preempted_.push_back(newest);
    ++n_preemptions_;
    return true;
}

const std::vector<PlanEntry>& Scheduler::plan() {
    std::set<int64_t> no_admit;           // preempted during this call: not admitted again in it
    for (;;) {
        for (const PlanEntry& e : plan_) cm_->rollback(e.id);
        plan_.clear();
        int budget = max_step_tokens_;
        bool again = false;

        // 1. one token for every request that is decoding
        int n_decoding = 0;
        for (size_t i = 0; i < running_.size() && !again; ++i) {
            const int64_t id = running_[i];
            const int cached = cm_->cached(id);
            if (reqs_[id].known - cached != 1) continue;
            ++n_decoding;
            if (budget < 1) continue;
            const int rc = cm_->reserve(id, 1);
            if (rc == -3) {
                const size_t before = preempted_.size();
                if (preempt_newest(id)) {
                    no_admit.insert(preempted_[before]);
                } else {
                    fail(id);             // alone and still no page: the context exceeds the pool
                }
                again = true;
                break;
            }
            plan_.push_back({id, cached, 1, 1});
            --budget;
        }
        if (again) continue;
        if (count_padded_rows_) {
            const int rows = (int)plan_.size();
            budget = std::max(0, budget - (padded_rows(rows) - rows));
        }

        // 2. the next portion of every prompt in flight
        auto fit = [&](int64_t id, int want, int spare) {
            // the largest n <= want whose pages are free in every group (keeping spare pages)
            std::vector<int> need(cm_->n_groups());
            auto fits = [&](int n) {
                cm_->pages_needed(id, n, need.data());
                for (int g = 0; g < cm_->n_groups(); ++g)
                    if (need[g] + spare > cm_->free_pages(g)) return false;
                return true;
            };
            if (fits(want)) return want;
            int lo = 0, hi = want;        // fits(lo) (0 tokens need nothing), !fits(hi)
            while (hi - lo > 1) {
                const int mid = (lo + hi) / 2;
                if (fits(mid)) lo = mid; else hi = mid;
            }
            return lo;
        };
        for (int64_t id : running_) {
            if (budget < 1) break;
            const int cached = cm_->cached(id);
            const int remaining = reqs_[id].known - cached;
            if (remaining <= 1) continue;
            const int n = fit(id, std::min(remaining, budget), 0);
            if (n < 1) continue;
            cm_->reserve(id, n);
            plan_.push_back({id, cached, n, cached + n == reqs_[id].known ? 1 : 0});
            budget -= n;
        }

        // 3. admit waiting requests, in order
        while (!waiting_.empty() && (int)running_.size() < max_running_ && cm_->free_slots() > 0 && budget > 0) {
            const int64_t id = waiting_.front();
            if (no_admit.count(id)) break;
            if (cm_->add_request(id) != 0) break;
            Req& r = reqs_[id];
            const int want = std::min(r.known, budget);
            int n;
            if (running_.empty()) {
                n = fit(id, want, 0);     // alone: take what fits
            } else {
                n = fit(id, want, n_decoding) == want ? want : 0;   // beside others: the portion plus a spare page per decoder
            }
            if (n < 1) {
                cm_->release(id);
                if (running_.empty()) { fail(id); again = true; }
                break;
            }
            waiting_.pop_front();
            r.order = next_order_++;
            running_.push_back(id);
            cm_->reserve(id, n);
            plan_.push_back({id, 0, n, n == r.known ? 1 : 0});
            budget -= n;
        }
        if (again) continue;

        // nothing could run although requests hold pages: make room
        if (plan_.empty() && !running_.empty()) {
            const size_t before = preempted_.size();
            if (preempt_newest(-1)) no_admit.insert(preempted_[before]);
            else fail(running_.front());
            continue;
        }
        // decode rows first, then portions: already in that order
        return plan_;
    }
}

void Scheduler::step_done(bool ok) {
    if (ok) {
        for (const PlanEntry& e : plan_) cm_->commit(e.id, e.count);
        ++n_steps_;
    } else {
        const std::vector<PlanEntry> entries = plan_;
        for (const PlanEntry& e : entries) fail(e.id);
    }
    plan_.clear();
}

int Scheduler::on_token(int64_t id, bool is_eos) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -1;
    Req& r = it->second;
    ++r.generated;
    if (!is_eos) ++r.known;
    if (is_eos || r.generated >= r.max_new || r.known >= max_context_) {
        cm_->release(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        reqs_.erase(it);
        return 1;
    }
    return 0;
}

int Scheduler::abort(int64_t id) {
    if (!reqs_.count(id)) return -1;
    for (const PlanEntry& e : plan_)
        if (e.id == id) return -2;        // in the step being run: abort after step_done
    cm_->release(id);
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    reqs_.erase(id);
    return 0;
}

std::vector<int64_t> Scheduler::take_preempted() {
    std::vector<int64_t> out;
    out.swap(preempted_);
    return out;
}

std::vector<int64_t> Scheduler::take_failed() {
    std::vector<int64_t> out;
    out.swap(failed_);
    return out;
}

int Scheduler::known_tokens(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -1 : it->second.known;
}

int Scheduler::generated(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -1 : it->second.generated;
}

}  // namespace imparo
