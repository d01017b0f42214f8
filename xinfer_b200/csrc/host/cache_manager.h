// Paged cache bookkeeping on the host: page pools per layer group, a block table per request
// and group, and the slots that index fixed-size per-request state.
//
// The reference keeps one pool of blocks with reference counts and a FIFO free list
// (src/core/block_manager.rs:19-56, 124-154) and one block table per sequence
// (src/core/sequence.rs:39).  Here every *group* of layers with the same needs (all keys, or a
// window of them) owns a pool and a table per request, pages are taken for exactly the tokens a
// step brings, and a windowed group gives pages back as soon as the window has passed them.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <utility>
#include <vector>

namespace xb {

struct GroupSpec {
    int page_size = 16;
    int num_pages = 0;
    int window = 0;  // <= 0: every earlier key is kept; else a query at p reads keys > p - window
};

// A pool of page ids, reused first-in first-out so that tests can predict which page comes next.
class PagePool {
public:
    explicit PagePool(int num_pages);
    int take();              // -1 when empty
    bool give(int page);     // false if the page is not held (double free, bad id)
    int free_count() const { return (int)free_.size(); }
    int size() const { return (int)held_.size(); }
    bool is_held(int page) const { return page >= 0 && page < (int)held_.size() && held_[page]; }

private:
    std::deque<int> free_;
    std::vector<uint8_t> held_;
};

class CacheManager {
public:
    CacheManager(const std::vector<GroupSpec>& groups, int max_requests);

    int num_groups() const { return (int)groups_.size(); }
    const GroupSpec& group(int g) const { return groups_[g]; }
    int max_requests() const { return (int)reqs_.size(); }

    // A slot for a new request (lowest free), or -1 when all are taken.
    int open_request();
    // Gives every page of the request back and frees the slot.  False if the slot is not live.
    bool close_request(int slot);
    bool is_live(int slot) const;
    int length(int slot) const;  // tokens whose keys/values are in the cache

    // Pages that growing the request to new_len tokens would take from group g.
    int pages_needed(int slot, int new_len, int g) const;
    bool can_extend(int slot, int new_len) const;
    // Takes the pages for tokens [length, new_len) in every group; all or nothing.
    bool extend(int slot, int new_len);
    // The step has written tokens up to new_len: record it and give back the pages of windowed
    // groups that no later query can read.
    bool advance(int slot, int new_len);

    int free_pages(int g) const { return pools_[g].free_count(); }
    // Entries of the request's table in group g (released pages read -1); returns their number.
    int table_size(int slot, int g) const;
    int copy_table(int slot, int g, int32_t* out, int capacity) const;
    int live_requests() const;

    // Debug aid: while on, every page that goes back to a pool is also written to a log, which the
    // owner of the device pages drains to overwrite them (stale contents must never be read).
    void log_freed(bool on) { log_freed_ = on; if (!on) freed_.clear(); }
    // Moves up to `capacity` (group, page) pairs of the log to `groups` / `pages`; returns how many.
    int drain_freed(int32_t* groups, int32_t* pages, int capacity);

    // Self-check for tests: every page is either free or held by exactly one table entry.
    bool consistent(std::string* why) const;

private:
    struct Request {
        bool live = false;
        int len = 0;
        std::vector<std::vector<int32_t>> tables;  // per group, indexed by position / page_size
    };
    int first_needed_page(int g, int len) const;
    bool log_freed_ = false;
    std::vector<std::pair<int32_t, int32_t>> freed_;

    std::vector<GroupSpec> groups_;
    std::vector<PagePool> pools_;
    std::vector<Request> reqs_;
};

}  // namespace xb
