#include "cache_manager.h"

#include <algorithm>
#include <sstream>

namespace xb {

PagePool::PagePool(int num_pages) : held_(num_pages > 0 ? num_pages : 0, 0) {
    for (int i = 0; i < num_pages; ++i) free_.push_back(i);
}

int PagePool::take() {
    if (free_.empty()) return -1;
    const int p = free_.front();
    free_.pop_front();
    held_[p] = 1;
    return p;
}

bool PagePool::give(int page) {
    if (!is_held(page)) return false;
    held_[page] = 0;
    free_.push_back(page);
    return true;
}

CacheManager::CacheManager(const std::vector<GroupSpec>& groups, int max_requests)
    : groups_(groups), reqs_(max_requests > 0 ? max_requests : 0) {
    for (const auto& g : groups_) pools_.emplace_back(g.num_pages);
    for (auto& r : reqs_) r.tables.resize(groups_.size());
}

int CacheManager::open_request() {
    for (int s = 0; s < (int)reqs_.size(); ++s) {
        if (!reqs_[s].live) {
            reqs_[s].live = true;
            reqs_[s].len = 0;
            for (auto& t : reqs_[s].tables) t.clear();
            return s;
        }
    }
    return -1;
}

bool CacheManager::is_live(int slot) const {
    return slot >= 0 && slot < (int)reqs_.size() && reqs_[slot].live;
}

int CacheManager::length(int slot) const { return is_live(slot) ? reqs_[slot].len : -1; }

bool CacheManager::close_request(int slot) {
    if (!is_live(slot)) return false;
    Request& r = reqs_[slot];
    bool ok = true;
    for (int g = 0; g < (int)groups_.size(); ++g) {
        // newest first, so the oldest pages of a finished request are reused last
        for (auto it = r.tables[g].rbegin(); it != r.tables[g].rend(); ++it)
            if (*it >= 0) {
                const bool gave = pools_[g].give(*it);
                if (gave && log_freed_) freed_.emplace_back(g, *it);
                ok = gave && ok;
            }
        r.tables[g].clear();
    }
    r.live = false;
    r.len = 0;
    return ok;
}

// First page index that a query at position >= len can still read in group g.
int CacheManager::first_needed_page(int g, int len) const {
    const GroupSpec& s = groups_[g];
    if (s.window <= 0) return 0;
    const int first_key = len - s.window + 1;
    return first_key > 0 ? first_key / s.page_size : 0;
}

int CacheManager::pages_needed(int slot, int new_len, int g) const {
    if (!is_live(slot)) return -1;
    const Request& r = reqs_[slot];
    const int ps = groups_[g].page_size;
    const int want = (new_len + ps - 1) / ps;
    const int have = (int)r.tables[g].size();
    return want > have ? want - have : 0;
}

bool CacheManager::can_extend(int slot, int new_len) const {
    if (!is_live(slot) || new_len < reqs_[slot].len) return false;
    for (int g = 0; g < (int)groups_.size(); ++g)
        if (pages_needed(slot, new_len, g) > pools_[g].free_count()) return false;
    return true;
}

bool CacheManager::extend(int slot, int new_len) {
    if (!can_extend(slot, new_len)) return false;
    Request& r = reqs_[slot];
    for (int g = 0; g < (int)groups_.size(); ++g) {
        const int n = pages_needed(slot, new_len, g);
        for (int i = 0; i < n; ++i) r.tables[g].push_back(pools_[g].take());
    }
    return true;
}

bool CacheManager::advance(int slot, int new_len) {
    if (!is_live(slot)) return false;
    Request& r = reqs_[slot];
    if (new_len < r.len) return false;
    for (int g = 0; g < (int)groups_.size(); ++g) {
        const int ps = groups_[g].page_size;
        if ((new_len + ps - 1) / ps > (int)r.tables[g].size()) return false;  // pages were never taken
    }
    r.len = new_len;
    for (int g = 0; g < (int)groups_.size(); ++g) {
        const int keep_from = std::min(first_needed_page(g, new_len), (int)r.tables[g].size());
        for (int i = 0; i < keep_from; ++i) {
            if (r.tables[g][i] >= 0) {
                if (pools_[g].give(r.tables[g][i]) && log_freed_) freed_.emplace_back(g, r.tables[g][i]);
                r.tables[g][i] = -1;
            }
        }
    }
    return true;
}

int CacheManager::drain_freed(int32_t* groups, int32_t* pages, int capacity) {
    const int n = std::min((int)freed_.size(), capacity);
    for (int i = 0; i < n; ++i) {
        groups[i] = freed_[i].first;
        pages[i] = freed_[i].second;
    }
    freed_.erase(freed_.begin(), freed_.begin() + n);
    return n;
}

int CacheManager::table_size(int slot, int g) const {
    return is_live(slot) ? (int)reqs_[slot].tables[g].size() : -1;
}

int CacheManager::copy_table(int slot, int g, int32_t* out, int capacity) const {
    if (!is_live(slot)) return -1;
    const auto& t = reqs_[slot].tables[g];
    const int n = std::min((int)t.size(), capacity);
    for (int i = 0; i < n; ++i) out[i] = t[i];
    return n;
}

int CacheManager::live_requests() const {
    int n = 0;
    for (const auto& r : reqs_) n += r.live ? 1 : 0;
    return n;
}

bool CacheManager::consistent(std::string* why) const {
    for (int g = 0; g < (int)groups_.size(); ++g) {
        std::vector<int> owners(pools_[g].size(), 0);
        for (const auto& r : reqs_) {
            if (!r.live) {
                if (!r.tables[g].empty()) {
                    if (why) *why = "a closed request still has a table";
                    return false;
                }
                continue;
            }
            for (int p : r.tables[g]) {
                if (p < 0) continue;
                if (p >= pools_[g].size()) {
                    if (why) *why = "a table holds a page id outside the pool";
                    return false;
                }
                owners[p]++;
            }
        }
        int held = 0;
        for (int p = 0; p < pools_[g].size(); ++p) {
            if (owners[p] > 1) {
                std::ostringstream s;
                s << "page " << p << " of group " << g << " is held by " << owners[p] << " table entries";
                if (why) *why = s.str();
                return false;
            }
            if (owners[p] == 1 && !pools_[g].is_held(p)) {
                if (why) *why = "a table holds a page that the pool counts as free";
                return false;
            }
            if (owners[p] == 0 && pools_[g].is_held(p)) {
                std::ostringstream s;
                s << "page " << p << " of group " << g << " is lost: held by the pool, in no table";
                if (why) *why = s.str();
                return false;
            }
            held += owners[p];
        }
        if (held + pools_[g].free_count() != pools_[g].size()) {
            if (why) *why = "held + free != pool size";
            return false;
        }
    }
    return true;
}

}  // namespace xb
