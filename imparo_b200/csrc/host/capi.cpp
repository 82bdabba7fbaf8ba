// C entry points of the host runtime, called from Python through ctypes.
#include <cstring>
#include <string>

#include "cache_manager.hpp"
#include "scheduler.hpp"

using imparo::CacheManager;
using imparo::GroupSpec;
using imparo::Scheduler;

extern "C" {

void* imparo_cm_create(int n_groups, const int* page_size, const int* n_pages, const int* window, int n_slots) {
    std::vector<GroupSpec> groups;
    for (int g = 0; g < n_groups; ++g) {
        if (page_size[g] < 1 || n_pages[g] < 0 || window[g] < 0) return nullptr;
        groups.push_back({page_size[g], n_pages[g], window[g]});
    }
    if (n_slots < 0) return nullptr;
    return new CacheManager(groups, n_slots);
}
void imparo_cm_destroy(void* cm) { delete static_cast<CacheManager*>(cm); }
int imparo_cm_add_request(void* cm, int64_t id) { return static_cast<CacheManager*>(cm)->add_request(id); }
int imparo_cm_pages_needed(void* cm, int64_t id, int n, int* per_group) { return static_cast<CacheManager*>(cm)->pages_needed(id, n, per_group); }
int imparo_cm_reserve(void* cm, int64_t id, int n) { return static_cast<CacheManager*>(cm)->reserve(id, n); }
int imparo_cm_commit(void* cm, int64_t id, int n) { return static_cast<CacheManager*>(cm)->commit(id, n); }
int imparo_cm_rollback(void* cm, int64_t id) { return static_cast<CacheManager*>(cm)->rollback(id); }
int imparo_cm_release(void* cm, int64_t id) { return static_cast<CacheManager*>(cm)->release(id); }
int imparo_cm_free_pages(void* cm, int group) { return static_cast<CacheManager*>(cm)->free_pages(group); }
int imparo_cm_free_slots(void* cm) { return static_cast<CacheManager*>(cm)->free_slots(); }
int imparo_cm_slot(void* cm, int64_t id) { return static_cast<CacheManager*>(cm)->slot(id); }
int imparo_cm_cached(void* cm, int64_t id) { return static_cast<CacheManager*>(cm)->cached(id); }
int imparo_cm_n_requests(void* cm) { return static_cast<CacheManager*>(cm)->n_requests(); }
int imparo_cm_table(void* cm, int64_t id, int group, int32_t* out, int max_blocks) { return static_cast<CacheManager*>(cm)->table(id, group, out, max_blocks); }
int imparo_cm_blocks_in_use(void* cm, int64_t id, int group) { return static_cast<CacheManager*>(cm)->blocks_in_use(id, group); }
int imparo_cm_check(void* cm, char* msg, int cap) {
    std::string err;
    const int rc = static_cast<CacheManager*>(cm)->check(&err);
    if (msg && cap > 0) { std::strncpy(msg, err.c_str(), cap - 1); msg[cap - 1] = 0; }
    return rc;
}

void* imparo_sched_create(void* cm, int max_step_tokens, int max_running, int max_context) {
    return new Scheduler(static_cast<CacheManager*>(cm), max_step_tokens, max_running, max_context);
}
void imparo_sched_destroy(void* s) { delete static_cast<Scheduler*>(s); }
void imparo_sched_count_padded_rows(void* s, int on) { static_cast<Scheduler*>(s)->count_padded_rows(on != 0); }
int imparo_padded_rows(int n) { return imparo::padded_rows(n); }
int64_t imparo_sched_submit(void* s, int prompt_len, int max_new) { return static_cast<Scheduler*>(s)->submit(prompt_len, max_new); }
int imparo_sched_plan(void* s, int64_t* ids, int* start, int* count, int* want, int cap) {
    const auto& p = static_cast<Scheduler*>(s)->plan();
    if ((int)p.size() > cap) return -1;
    for (size_t i = 0; i < p.size(); ++i) { ids[i] = p[i].id; start[i] = p[i].start; count[i] = p[i].count; want[i] = p[i].want; }
    return (int)p.size();
}
void imparo_sched_step_done(void* s, int ok) { static_cast<Scheduler*>(s)->step_done(ok != 0); }
int imparo_sched_on_token(void* s, int64_t id, int is_eos) { return static_cast<Scheduler*>(s)->on_token(id, is_eos != 0); }
int imparo_sched_abort(void* s, int64_t id) { return static_cast<Scheduler*>(s)->abort(id); }
int imparo_sched_has_work(void* s) { return static_cast<Scheduler*>(s)->has_work() ? 1 : 0; }
int imparo_sched_n_waiting(void* s) { return static_cast<Scheduler*>(s)->n_waiting(); }
int imparo_sched_n_running(void* s) { return static_cast<Scheduler*>(s)->n_running(); }
int64_t imparo_sched_n_preemptions(void* s) { return static_cast<Scheduler*>(s)->n_preemptions(); }
int64_t imparo_sched_n_steps(void* s) { return static_cast<Scheduler*>(s)->n_steps(); }
int imparo_sched_known_tokens(void* s, int64_t id) { return static_cast<Scheduler*>(s)->known_tokens(id); }
int imparo_sched_generated(void* s, int64_t id) { return static_cast<Scheduler*>(s)->generated(id); }
static int drain(const std::vector<int64_t>& v, int64_t* out, int cap) {
    const int n = std::min((int)v.size(), cap);
    for (int i = 0; i < n; ++i) out[i] = v[i];
    return n;
}
int imparo_sched_take_preempted(void* s, int64_t* out, int cap) { return drain(static_cast<Scheduler*>(s)->take_preempted(), out, cap); }
int imparo_sched_take_failed(void* s, int64_t* out, int cap) { return drain(static_cast<Scheduler*>(s)->take_failed(), out, cap); }

}  // extern "C"
