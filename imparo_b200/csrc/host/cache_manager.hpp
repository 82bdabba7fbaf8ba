// Cache bookkeeping on the host: pages with a block table per request, per group of
// layers, and fixed-size state slots.  It deals in page and slot numbers only; the
// device arenas they index are owned by the Python side.
//
// What the reference does and this keeps: the lowest free block is always handed out, so
// what a request gets depends on the free set alone, never on history
// (imparo-kv/src/alloc.rs:1-11,55-69); a position's row is table[pos / page] * page +
// pos % page (imparo-cuda/native/kv_paging.cuh:25-30); layers that keep every position
// and layers that keep a window are different kinds of state (imparo-kv/src/state.rs:16-21);
// a request takes pages as it grows, not up front (imparo-server/src/sched.rs:671-696);
// recurrent state lives in a per-conversation slot that starts from zero
// (imparo-model/src/lib.rs:1951-1972).  What differs: pages go back to the free set the
// moment a request ends or a window has passed them (there is no prefix store).
#pragma once
#include <cstdint>
#include <map>
#include <set>
#include <string>
#include <vector>

namespace imparo {

struct GroupSpec {
    int page_size;
    int n_pages;
    int window;   // 0: keep every position
};

class CacheManager {
public:
    CacheManager(const std::vector<GroupSpec>& groups, int n_slots);

    // 0, or -1 (request exists), -2 (no state slot free).  The slot is the lowest free one.
    int add_request(int64_t id);
    // Pages that appending n tokens would take, per group (nullptr allowed); -1 unknown id.
    int pages_needed(int64_t id, int n_tokens, int* per_group) const;
    // Map positions [cached, cached+n) in every group; all groups or none.
    // 0, -1 unknown id, -3 not enough free pages, -4 bad n.
    int reserve(int64_t id, int n_tokens);
    // The step ran: cached += n.  Pages a window has passed go back.  n must be reserved.
    int commit(int64_t id, int n_tokens);
    // Undo a reserve whose step did not run: pages beyond what cached needs go back.
    int rollback(int64_t id);
    // Everything the request holds goes back.
    int release(int64_t id);

    int free_pages(int group) const;
    int free_slots() const { return (int)free_slots_.size(); }
    int n_groups() const { return (int)groups_.size(); }
    int slot(int64_t id) const;
    int cached(int64_t id) const;
    int n_requests() const { return (int)requests_.size(); }
    // Block table of one request in one group: out[b] = page or -1; returns blocks written.
    int table(int64_t id, int group, int32_t* out, int max_blocks) const;
    int blocks_in_use(int64_t id, int group) const;
    // Invariants: every page is free or held by exactly one request, every slot likewise.
    // 0 when they hold; else a code, with a description in error.
    int check(std::string* error) const;

private:
    struct Request {
        int slot = -1;
        int cached = 0;
        int reserved = 0;                           // tokens mapped beyond cached
        std::vector<std::vector<int32_t>> tables;   // per group: block -> page or -1
    };
    int first_block_needed(const GroupSpec& g, int next_pos) const;
    void trim(Request& r, int upto_tokens);

    std::vector<GroupSpec> groups_;
    std::vector<std::set<int32_t>> free_pages_;
    std::set<int32_t> free_slots_;
    int n_slots_;
    std::map<int64_t, Request> requests_;
};

}  // namespace imparo
