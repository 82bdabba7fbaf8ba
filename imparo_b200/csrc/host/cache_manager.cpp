#include "cache_manager.hpp"

#include <algorithm>
#include <cstring>

namespace imparo {

CacheManager::CacheManager(const std::vector<GroupSpec>& groups, int n_slots)
    : groups_(groups), free_pages_(groups.size()), n_slots_(n_slots) {
    for (size_t g = 0; g < groups_.size(); ++g)
        for (int p = 0; p < groups_[g].n_pages; ++p) free_pages_[g].insert(p);
    for (int s = 0; s < n_slots; ++s) free_slots_.insert(s);
}

int CacheManager::first_block_needed(const GroupSpec& g, int next_pos) const {
    if (g.window <= 0) return 0;
    const int lo = std::max(0, next_pos + 1 - g.window);
    return lo / g.page_size;
}

int CacheManager::add_request(int64_t id) {
    if (requests_.count(id)) return -1;
    if (free_slots_.empty()) return -2;
    Request r;
    r.slot = *free_slots_.begin();
    free_slots_.erase(free_slots_.begin());
    r.tables.resize(groups_.size());
    requests_.emplace(id, std::move(r));
    return 0;
}

int CacheManager::pages_needed(int64_t id, int n_tokens, int* per_group) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) return -1;
    const Request& r = it->second;
    int total = 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        int need = 0;
        if (n_tokens > 0) {
            const int first = first_block_needed(groups_[g], r.cached);
            const int last = (r.cached + n_tokens - 1) / groups_[g].page_size;
            const auto& tab = r.tables[g];
            for (int b = first; b <= last; ++b)
                if (b >= (int)tab.size() || tab[b] < 0) ++need;
        }
        if (per_group) per_group[g] = need;
        total += need;
    }
    return total;
}

int CacheManager::reserve(int64_t id, int n_tokens) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return -1;
    if (n_tokens <= 0) return -4;
    Request& r = it->second;
    std::vector<int> need(groups_.size());
    pages_needed(id, n_tokens, need.data());
    for (size_t g = 0; g < groups_.size(); ++g)
        if (need[g] > (int)free_pages_[g].size()) return -3;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int first = first_block_needed(groups_[g], r.cached);
        const int last = (r.cached + n_tokens - 1) / groups_[g].page_size;
        auto& tab = r.tables[g];
        if ((int)tab.size() <= last) tab.resize(last + 1, -1);
        for (int b = first; b <= last; ++b) {
            if (tab[b] >= 0) continue;
            tab[b] = *free_pages_[g].begin();          // the lowest free page
            free_pages_[g].erase(free_pages_[g].begin());
        }
    }
    r.reserved = std::max(r.reserved, n_tokens);
    return 0;
}

void CacheManager::trim(Request& r, int upto_tokens) {
    // give back every page beyond what upto_tokens positions need
    for (size_t g = 0; g < groups_.size(); ++g) {
        auto& tab = r.tables[g];
        const int keep = (upto_tokens + groups_[g].page_size - 1) / groups_[g].page_size;
        for (int b = keep; b < (int)tab.size(); ++b)
            if (tab[b] >= 0) { free_pages_[g].insert(tab[b]); tab[b] = -1; }
        if ((int)tab.size() > keep) tab.resize(keep);
    }
}

int CacheManager::commit(int64_t id, int n_tokens) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return -1;
    Request& r = it->second;
    if (n_tokens <= 0 || n_tokens > r.reserved) return -4;
    r.cached += n_tokens;
    r.reserved = 0;
    trim(r, r.cached);
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int first = first_block_needed(groups_[g], r.cached);
        auto& tab = r.tables[g];
        for (int b = 0; b < first && b < (int)tab.size(); ++b)
            if (tab[b] >= 0) { free_pages_[g].insert(tab[b]); tab[b] = -1; }
    }
    return 0;
}

int CacheManager::rollback(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return -1;
    it->second.reserved = 0;
    trim(it->second, it->second.cached);
    return 0;
}

int CacheManager::release(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) return -1;
    Request& r = it->second;
    for (size_t g = 0; g < groups_.size(); ++g)
        for (int32_t p : r.tables[g])
            if (p >= 0) free_pages_[g].insert(p);
    free_slots_.insert(r.slot);
    requests_.erase(it);
    return 0;
}

int CacheManager::free_pages(int group) const {
    if (group < 0 || group >= (int)groups_.size()) return -1;
    return (int)free_pages_[group].size();
}

int CacheManager::slot(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? -1 : it->second.slot;
}

int CacheManager::cached(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? -1 : it->second.cached;
}

int CacheManager::table(int64_t id, int group, int32_t* out, int max_blocks) const {
    auto it = requests_.find(id);
    if (it == requests_.end() || group < 0 || group >= (int)groups_.size()) return -1;
    const auto& tab = it->second.tables[group];
    const int n = std::min((int)tab.size(), max_blocks);
    for (int b = 0; b < n; ++b) out[b] = tab[b];
    return (int)tab.size();
}

int CacheManager::blocks_in_use(int64_t id, int group) const {
    auto it = requests_.find(id);
    if (it == requests_.end() || group < 0 || group >= (int)groups_.size()) return -1;
    int n = 0;
    for (int32_t p : it->second.tables[group]) n += p >= 0;
    return n;
}

int CacheManager::check(std::string* error) const {
    auto fail = [&](int code, const std::string& msg) { if (error) *error = msg; return code; };
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::vector<int> holders(groups_[g].n_pages, 0);
        for (int32_t p : free_pages_[g]) {
            if (p < 0 || p >= groups_[g].n_pages) return fail(1, "free set holds a page out of range");
            holders[p]++;
        }
        for (const auto& kv : requests_)
            for (int32_t p : kv.second.tables[g]) {
                if (p < 0) continue;
                if (p >= groups_[g].n_pages) return fail(2, "a table holds a page out of range");
                holders[p]++;
            }
        for (int p = 0; p < groups_[g].n_pages; ++p) {
            if (holders[p] == 0) return fail(3, "page " + std::to_string(p) + " of group " + std::to_string(g) + " is lost");
            if (holders[p] > 1) return fail(4, "page " + std::to_string(p) + " of group " + std::to_string(g) + " is held twice");
        }
    }
    std::vector<int> holders(n_slots_, 0);
    for (int32_t s : free_slots_) holders[s]++;
    for (const auto& kv : requests_) {
        if (kv.second.slot < 0 || kv.second.slot >= n_slots_) return fail(5, "a request holds a slot out of range");
        holders[kv.second.slot]++;
    }
    for (int s = 0; s < n_slots_; ++s) {
        if (holders[s] == 0) return fail(6, "slot " + std::to_string(s) + " is lost");
        if (holders[s] > 1) return fail(7, "slot " + std::to_string(s) + " is held twice");
    }
    return 0;
}

}  // namespace imparo
