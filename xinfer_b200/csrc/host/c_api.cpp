// C interface of the host runtime (loaded from Python with ctypes): cache manager, scheduler and
// the assembly of a step's metadata into one packed int32 buffer that a single copy sends to the
// device.
#include <algorithm>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#include "cache_manager.h"
#include "scheduler.h"

#define XB_API extern "C" __attribute__((visibility("default")))

using namespace xb;

// ---- cache manager -------------------------------------------------------------------------
XB_API void* xb_cm_create(int n_groups, const int* page_sizes, const int* num_pages, const int* windows,
                          int max_requests) {
    if (n_groups <= 0 || max_requests <= 0) return nullptr;
    std::vector<GroupSpec> groups(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        if (page_sizes[g] <= 0 || num_pages[g] <= 0) return nullptr;
        groups[g].page_size = page_sizes[g];
        groups[g].num_pages = num_pages[g];
        groups[g].window = windows[g];
    }
    return new CacheManager(groups, max_requests);
}
XB_API void xb_cm_destroy(void* h) { delete static_cast<CacheManager*>(h); }
XB_API int xb_cm_open(void* h) { return static_cast<CacheManager*>(h)->open_request(); }
XB_API int xb_cm_close(void* h, int slot) { return static_cast<CacheManager*>(h)->close_request(slot) ? 1 : 0; }
XB_API int xb_cm_is_live(void* h, int slot) { return static_cast<CacheManager*>(h)->is_live(slot) ? 1 : 0; }
XB_API int xb_cm_length(void* h, int slot) { return static_cast<CacheManager*>(h)->length(slot); }
XB_API int xb_cm_can_extend(void* h, int slot, int new_len) { return static_cast<CacheManager*>(h)->can_extend(slot, new_len) ? 1 : 0; }
XB_API int xb_cm_extend(void* h, int slot, int new_len) { return static_cast<CacheManager*>(h)->extend(slot, new_len) ? 1 : 0; }
XB_API int xb_cm_advance(void* h, int slot, int new_len) { return static_cast<CacheManager*>(h)->advance(slot, new_len) ? 1 : 0; }
XB_API int xb_cm_free_pages(void* h, int g) { return static_cast<CacheManager*>(h)->free_pages(g); }
XB_API int xb_cm_table_size(void* h, int slot, int g) { return static_cast<CacheManager*>(h)->table_size(slot, g); }
XB_API int xb_cm_copy_table(void* h, int slot, int g, int32_t* out, int cap) { return static_cast<CacheManager*>(h)->copy_table(slot, g, out, cap); }
XB_API int xb_cm_live_requests(void* h) { return static_cast<CacheManager*>(h)->live_requests(); }
XB_API void xb_cm_log_freed(void* h, int on) { static_cast<CacheManager*>(h)->log_freed(on != 0); }
XB_API int xb_cm_drain_freed(void* h, int32_t* groups, int32_t* pages, int cap) {
    return static_cast<CacheManager*>(h)->drain_freed(groups, pages, cap);
}
XB_API int xb_cm_consistent(void* h, char* why, int cap) {
    std::string s;
    const bool ok = static_cast<CacheManager*>(h)->consistent(&s);
    if (why && cap > 0) {
        std::strncpy(why, s.c_str(), cap - 1);
        why[cap - 1] = 0;
    }
    return ok ? 1 : 0;
}

// ---- step metadata ---------------------------------------------------------------------------
// Packs, for B entries (slot, count, tokens) whose start is the slot's cached length:
//   token_ids[Tp] positions[Tp] req_of_token[Tp] q_start[Bp+1] start_pos[Bp] slots[Bp]
//   logit_rows[Rp] and, per group, block_table[Bp, stride_g]
// Tp/Bp/Rp are T, B and R padded up to pad_tokens / pad_entries / pad_rows (padding rows read
// row 0; padding tokens belong to request -1
// and are skipped by the kernels); every array starts on a 16-byte boundary.  `strides` holds a
// wanted row length per group (0: as long as the longest table here, rounded up to 8).
// offsets_out[0..6] = array offsets in int32 units, [7 + g] = table offset of group g,
// [7 + G + g] = stride of group g, and the return value is the number of int32 used
// (negative on error: -1 capacity, -2 slot not live, -3 pages missing, -4 bad want).
XB_API long long xb_assemble(void* h, int B, const int* slots, const int* counts, const int* tokens,
                             int R, const int* want_entry, const int* want_offset, int pad_tokens,
                             int pad_entries, int pad_rows, const int* strides, int32_t* out, long long capacity,
                             long long* offsets_out) {
    CacheManager* cm = static_cast<CacheManager*>(h);
    const int G = cm->num_groups();
    int T = 0;
    for (int b = 0; b < B; ++b) {
        if (!cm->is_live(slots[b]) || counts[b] <= 0) return -2;
        T += counts[b];
    }
    const int Tp = std::max(T, pad_tokens), Bp = std::max(B, pad_entries), Rp = std::max(std::max(R, pad_rows), 1);
    auto up4 = [](long long x) { return (x + 3) / 4 * 4; };
    std::vector<int> stride(G);
    for (int g = 0; g < G; ++g) {
        int longest = 1;
        const int ps = cm->group(g).page_size;
        for (int b = 0; b < B; ++b) {
            const int new_len = cm->length(slots[b]) + counts[b];
            if (cm->table_size(slots[b], g) * ps < new_len) return -3;
            longest = std::max(longest, (new_len + ps - 1) / ps);
        }
        stride[g] = (longest + 7) / 8 * 8;
        if (strides && strides[g] > 0) {
            if (strides[g] < longest) return -1;
            stride[g] = strides[g];
        }
    }
    long long off = 0;
    long long o_tok = off; off = up4(off + Tp);
    long long o_pos = off; off = up4(off + Tp);
    long long o_req = off; off = up4(off + Tp);
    long long o_qs = off; off = up4(off + Bp + 1);
    long long o_sp = off; off = up4(off + Bp);
    long long o_sl = off; off = up4(off + Bp);
    long long o_rows = off; off = up4(off + Rp);
    std::vector<long long> o_tab(G);
    for (int g = 0; g < G; ++g) {
        o_tab[g] = off;
        off = up4(off + (long long)Bp * stride[g]);
    }
    if (off > capacity) return -1;
    int t = 0;
    for (int b = 0; b < B; ++b) {
        const int start = cm->length(slots[b]);
        out[o_qs + b] = t;
        out[o_sp + b] = start;
        out[o_sl + b] = slots[b];
        for (int i = 0; i < counts[b]; ++i, ++t) {
            out[o_tok + t] = tokens[t];
            out[o_pos + t] = start + i;
            out[o_req + t] = b;
        }
    }
    for (int b = B; b <= Bp; ++b) out[o_qs + b] = T;
    for (int b = B; b < Bp; ++b) {
        out[o_sp + b] = 0;
        out[o_sl + b] = -1;
    }
    for (; t < Tp; ++t) {
        out[o_tok + t] = 0;
        out[o_pos + t] = 0;
        out[o_req + t] = -1;
    }
    for (int r = 0; r < R; ++r) {
        const int e = want_entry[r];
        if (e < 0 || e >= B || want_offset[r] < 0 || want_offset[r] >= counts[e]) return -4;
        out[o_rows + r] = out[o_qs + e] + want_offset[r];
    }
    for (int r = R; r < Rp; ++r) out[o_rows + r] = 0;
    for (int g = 0; g < G; ++g) {
        for (int b = 0; b < Bp; ++b) {
            int32_t* row = out + o_tab[g] + (long long)b * stride[g];
            int n = 0;
            if (b < B) n = cm->copy_table(slots[b], g, row, stride[g]);
            for (int i = std::max(n, 0); i < stride[g]; ++i) row[i] = -1;
        }
    }
    offsets_out[0] = o_tok; offsets_out[1] = o_pos; offsets_out[2] = o_req; offsets_out[3] = o_qs;
    offsets_out[4] = o_sp; offsets_out[5] = o_sl; offsets_out[6] = o_rows;
    for (int g = 0; g < G; ++g) {
        offsets_out[7 + g] = o_tab[g];
        offsets_out[7 + G + g] = stride[g];
    }
    return off;
}

// ---- work lists of the prefill attention kernel ---------------------------------------------------
// The step's portions of more than dec_max tokens are cut into items of 128 queries (a query tile) of
// two query heads that share a key/value head (one head where a group has an odd head left); an item's
// cost is its number of 64-key tiles times the cost of a tile (of two heads, or of one) plus a fixed
// start-up.  The items go, longest first, each onto the CTA with the least work so far, so that all CTAs
// end together whatever the portions' lengths are; items of equal cost - the heads of one query tile,
// which read the same keys - land on different CTAs and run at the same time.  The same is tried with
// one head per item (twice the items, each two thirds as long), and the cut that ends earlier is taken:
// one head where two-head items would leave CTAs idle (short portions, few heads), two otherwise.
// out: [ctas + 1] offsets (in items) then 4 int32 per item: portion, query tile, first query head, heads.
// Returns the number of int32 written (-1: capacity too small) and the number of CTAs in *ctas_out.
XB_API long long xb_attn_prefill_work(int B, const int* counts, const int* starts, int dec_max, int window,
                                      int heads, int kv_heads, int max_ctas, int32_t* out, long long capacity,
                                      int* ctas_out) {
    // costs in sixths of a key tile of two heads: a tile of one head takes about two thirds of the time of a tile
    // of two (measured at long contexts: 0.76 us against 1.15 us), an item's start about three tiles
    constexpr int QT = 128, KT = 64, TILE_OF_TWO = 6, TILE_OF_ONE = 4, START_UP = 18, INTS = 4;
    struct Tile { int tiles, b, tile; };
    std::vector<Tile> tiles;
    for (int b = 0; b < B; ++b) {
        const int n = counts[b];
        if (n <= dec_max) continue;
        for (int ti = 0; ti * QT < n; ++ti) {
            const int p0 = starts[b] + ti * QT, rows = std::min(QT, n - ti * QT);
            const int last_key = p0 + rows - 1, first_key = window > 0 ? std::max(0, p0 - window + 1) : 0;
            tiles.push_back({last_key / KT - first_key / KT + 1, b, ti});
        }
    }
    *ctas_out = 0;
    if (tiles.empty() || heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& x, const Tile& y) { return x.tiles > y.tiles; });
    const int G = heads / kv_heads, per_group = (G + 1) / 2;
    struct Head { int h0, nhd; };
    struct Shared { std::vector<std::vector<int32_t>> lists; long long longest = 0, n_items = 0; };
    // items of two heads (`singles` false) or of one, shared out: least loaded CTA first, ties to the lower index
    auto share_out = [&](bool singles, Shared& made) {
        std::vector<Head> head_items;
        for (int g = 0; g < kv_heads; ++g) {
            if (singles) {
                for (int h = 0; h < G; ++h) head_items.push_back({g * G + h, 1});
            } else {
                for (int pr = 0; pr < per_group; ++pr) head_items.push_back({g * G + 2 * pr, 2 * pr + 1 < G ? 2 : 1});
            }
        }
        made.n_items = (long long)tiles.size() * (long long)head_items.size();
        const int ctas = (int)std::min<long long>(max_ctas, made.n_items);
        std::vector<std::pair<long long, int>> heap;
        for (int c = 0; c < ctas; ++c) heap.emplace_back(0, c);
        auto later = [](const std::pair<long long, int>& x, const std::pair<long long, int>& y) { return x > y; };
        std::make_heap(heap.begin(), heap.end(), later);
        made.lists.assign(ctas, {});
        for (const Tile& t : tiles) {
            for (const Head& h : head_items) {
                std::pop_heap(heap.begin(), heap.end(), later);
                auto& top = heap.back();
                made.lists[top.second].insert(made.lists[top.second].end(), {t.b, t.tile, h.h0, h.nhd});
                top.first += (long long)t.tiles * (h.nhd == 2 ? TILE_OF_TWO : TILE_OF_ONE) + START_UP;
                made.longest = std::max(made.longest, top.first);
                std::push_heap(heap.begin(), heap.end(), later);
            }
        }
    };
    // two heads per item load a key/value tile once for both; one head per item gives twice as many items to
    // fill the CTAs with.  Whichever ends earlier by these costs is taken (a few thousand items at most).
    Shared made;
    share_out(false, made);
    if (G >= 2) {
        Shared ones;
        share_out(true, ones);
        if (ones.longest < made.longest) made = std::move(ones);
    }
    const std::vector<std::vector<int32_t>>& lists = made.lists;
    const long long n_items = made.n_items;
    const int ctas = (int)lists.size();
    *ctas_out = ctas;
    if ((long long)ctas + 1 + INTS * n_items > capacity) return -1;
    int32_t* items = out + ctas + 1;
    int at = 0;
    for (int c = 0; c < ctas; ++c) {
        out[c] = at;
        std::copy(lists[c].begin(), lists[c].end(), items + INTS * (long long)at);
        at += (int)lists[c].size() / INTS;
    }
    out[ctas] = at;
    return (long long)ctas + 1 + INTS * n_items;
}

// ---- scheduler ---------------------------------------------------------------------------------
struct SchedHandle {
    Scheduler sched;
    std::vector<StepEntry> last;    // scheduled, not yet committed
    std::vector<StepEntry> ahead;   // the step after `last`, decided while `last` runs
    SchedHandle(CacheManager* c, const SchedulerConfig& cfg) : sched(c, cfg) {}
};

XB_API void* xb_sched_create(void* cm, int max_num_seqs, int max_batched_tokens, int prefill_chunk,
                             int max_model_len, const int* eos_ids, int n_eos) {
    if (!cm || max_num_seqs <= 0 || max_batched_tokens <= 0 || prefill_chunk <= 0 || max_model_len <= 1) return nullptr;
    SchedulerConfig cfg;
    cfg.max_num_seqs = max_num_seqs;
    cfg.max_num_batched_tokens = max_batched_tokens;
    cfg.prefill_chunk_size = prefill_chunk;
    cfg.max_model_len = max_model_len;
    if (n_eos > 0) cfg.eos_token_ids.assign(eos_ids, eos_ids + n_eos);
    return new SchedHandle(static_cast<CacheManager*>(cm), cfg);
}
XB_API void xb_sched_destroy(void* h) { delete static_cast<SchedHandle*>(h); }
XB_API int xb_sched_add(void* h, long long req_id, const int* prompt, int n, int max_tokens, int ignore_eos,
                        const int* stop_ids, const int* stop_lens, int n_stop) {
    return (int)static_cast<SchedHandle*>(h)->sched.add(req_id, prompt, n, max_tokens, ignore_eos != 0, stop_ids, stop_lens, n_stop);
}
XB_API int xb_sched_abort(void* h, long long req_id) { return static_cast<SchedHandle*>(h)->sched.abort(req_id) ? 1 : 0; }

// Returns the number of entries (or -1 if the arrays are too small) and keeps them for commit.
XB_API int xb_sched_schedule(void* h, int cap_entries, long long* req_ids, int* slots, int* starts,
                             int* counts, int* wants, int cap_tokens, int* tokens, int* n_tokens) {
    SchedHandle* s = static_cast<SchedHandle*>(h);
    std::vector<int32_t> toks;
    s->last = s->sched.schedule(&toks);
    if ((int)s->last.size() > cap_entries || (int)toks.size() > cap_tokens) return -1;
    for (size_t i = 0; i < s->last.size(); ++i) {
        req_ids[i] = s->last[i].req_id;
        slots[i] = s->last[i].slot;
        starts[i] = s->last[i].start;
        counts[i] = s->last[i].count;
        wants[i] = s->last[i].want ? 1 : 0;
    }
    std::copy(toks.begin(), toks.end(), tokens);
    *n_tokens = (int)toks.size();
    return (int)s->last.size();
}
// Commits the oldest uncommitted step; a step decided ahead becomes the one awaiting commit.
XB_API void xb_sched_commit(void* h, const int* sampled, int n_sampled) {
    SchedHandle* s = static_cast<SchedHandle*>(h);
    std::vector<int32_t> v(sampled, sampled + (n_sampled > 0 ? n_sampled : 0));
    s->sched.commit(s->last, v);
    s->last.swap(s->ahead);
    s->ahead.clear();
}
// The step after the uncommitted one (see Scheduler::schedule_ahead).  Returns the number of
// entries, 0 when it cannot be decided ahead, -1 if the arrays are too small.
XB_API int xb_sched_schedule_ahead(void* h, int cap_entries, long long* req_ids, int* slots, int* starts, int* src) {
    SchedHandle* s = static_cast<SchedHandle*>(h);
    if (!s->ahead.empty()) return 0;
    std::vector<int> from;
    std::vector<StepEntry> e = s->sched.schedule_ahead(s->last, &from);
    if ((int)e.size() > cap_entries) return -1;
    for (size_t i = 0; i < e.size(); ++i) {
        req_ids[i] = e[i].req_id;
        slots[i] = e[i].slot;
        starts[i] = e[i].start;
        src[i] = from[i];
    }
    s->ahead = e;
    return (int)e.size();
}
// A scheduled step failed on the device or on the way there: every request of the steps that are
// scheduled and not committed (the running one and the one decided ahead) ends as aborted, its pages
// go back, and nothing stays scheduled.  Returns how many requests that ended.
XB_API int xb_sched_fail_steps(void* h) {
    SchedHandle* s = static_cast<SchedHandle*>(h);
    int n = 0;
    for (std::vector<StepEntry>* v : {&s->last, &s->ahead}) {
        for (const StepEntry& e : *v)
            if (s->sched.abort(e.req_id)) ++n;
        v->clear();
    }
    return n;
}
XB_API int xb_sched_drain_finished(void* h, long long* out, int cap) {
    auto v = static_cast<SchedHandle*>(h)->sched.drain_finished();
    const int n = std::min((int)v.size(), cap);
    for (int i = 0; i < n; ++i) out[i] = v[i];
    return n;
}
XB_API int xb_sched_num_waiting(void* h) { return static_cast<SchedHandle*>(h)->sched.num_waiting(); }
XB_API int xb_sched_num_running(void* h) { return static_cast<SchedHandle*>(h)->sched.num_running(); }
XB_API int xb_sched_preemptions(void* h) { return static_cast<SchedHandle*>(h)->sched.preemptions(); }
XB_API int xb_sched_finish_reason(void* h, long long id) { return static_cast<SchedHandle*>(h)->sched.finish_reason(id); }
XB_API int xb_sched_output_length(void* h, long long id) { return static_cast<SchedHandle*>(h)->sched.output_length(id); }
XB_API int xb_sched_copy_output(void* h, long long id, int* out, int cap) { return static_cast<SchedHandle*>(h)->sched.copy_output(id, out, cap); }
XB_API int xb_sched_prompt_length(void* h, long long id) { return static_cast<SchedHandle*>(h)->sched.prompt_length(id); }
XB_API int xb_sched_num_drawn(void* h, long long id) { return static_cast<SchedHandle*>(h)->sched.num_drawn(id); }
XB_API int xb_sched_copy_tail(void* h, long long id, int* out, int n) { return static_cast<SchedHandle*>(h)->sched.copy_tail(id, out, n); }
XB_API int xb_sched_release(void* h, long long id) { return static_cast<SchedHandle*>(h)->sched.release(id) ? 1 : 0; }
