#include "scheduler.h"

#include <algorithm>

namespace xb {

Scheduler::Scheduler(CacheManager* cache, const SchedulerConfig& cfg) : cache_(cache), cfg_(cfg) {}

AddStatus Scheduler::add(int64_t req_id, const int32_t* prompt, int n, int max_tokens,
                         bool ignore_eos, const int32_t* stop_ids, const int32_t* stop_lens, int n_stop) {
    if (n <= 0) return ADD_EMPTY_PROMPT;
    if (reqs_.count(req_id)) return ADD_DUPLICATE;
    // the reference refuses prompts longer than max_model_len - 1 and clips max_tokens so that
    // prompt + output fits (src/core/engine.rs:639-678)
    if (n > cfg_.max_model_len - 1) return ADD_TOO_LONG;
    if (max_tokens < 1) max_tokens = 1;
    max_tokens = std::min(max_tokens, cfg_.max_model_len - n);
    const int total = n + max_tokens;
    for (int g = 0; g < cache_->num_groups(); ++g) {
        const GroupSpec& s = cache_->group(g);
        int most = total;
        if (s.window > 0) {
            // a windowed group holds at most one portion plus the window behind it
            const int portion = std::min(std::min(cfg_.prefill_chunk_size, cfg_.max_num_batched_tokens), n);
            most = std::min(total, s.window + portion + s.page_size);
        }
        if ((most + s.page_size - 1) / s.page_size > s.num_pages) return ADD_NEVER_FITS;
    }
    Request r;
    r.id = req_id;
    r.tokens.assign(prompt, prompt + n);
    r.prompt_len = n;
    r.max_tokens = max_tokens;
    r.ignore_eos = ignore_eos;
    for (int i = 0, at = 0; i < n_stop; ++i) {
        const int len = stop_lens ? stop_lens[i] : 1;
        if (len > 0) r.stop_seqs.emplace_back(stop_ids + at, stop_ids + at + len);
        at += std::max(len, 0);
    }
    reqs_[req_id] = std::move(r);
    waiting_.push_back(req_id);
    return ADD_OK;
}

void Scheduler::finish(Request& r, int reason) {
    r.finish = reason;
    finished_.push_back(r.id);
    if (r.slot >= 0) {
        cache_->close_request(r.slot);
        r.slot = -1;
    }
    running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r.id), waiting_.end());
}

bool Scheduler::abort(int64_t req_id) {
    auto it = reqs_.find(req_id);
    if (it == reqs_.end() || it->second.finish != NOT_FINISHED) return false;
    finish(it->second, FINISH_ABORT);
    return true;
}

void Scheduler::preempt_newest() {
    if (running_.empty()) return;
    Request& v = reqs_[running_.back()];
    running_.pop_back();
    cache_->close_request(v.slot);
    v.slot = -1;
    v.computed = 0;
    waiting_.push_front(v.id);
    ++preemptions_;
}

// Largest n' <= n such that growing `slot` from `computed` by n' tokens finds its pages.
static int fit_tokens(const CacheManager& c, int slot, int computed, int n) {
    for (int g = 0; g < c.num_groups(); ++g) {
        const int ps = c.group(g).page_size;
        const long long room = (long long)(c.table_size(slot, g) + c.free_pages(g)) * ps - computed;
        if (room < n) n = (int)std::max<long long>(room, 0);
    }
    return n;
}

std::vector<StepEntry> Scheduler::schedule(std::vector<int32_t>* tokens) {
    std::vector<StepEntry> entries;
    tokens->clear();
    for (;;) {
        entries.clear();
        tokens->clear();
        int budget = cfg_.max_num_batched_tokens;
        bool preempted = false;
        auto push = [&](Request& r, int n) {
            StepEntry e;
            e.req_id = r.id;
            e.slot = r.slot;
            e.start = r.computed;
            e.count = n;
            e.want = r.computed + n == (int)r.tokens.size();
            entries.push_back(e);
            tokens->insert(tokens->end(), r.tokens.begin() + r.computed, r.tokens.begin() + r.computed + n);
            budget -= n;
        };
        // 1. one token for every request that is decoding; a decode that finds no page makes the
        //    newest running request give its pages back
        for (size_t i = 0; i < running_.size() && budget > 0;) {
            Request& r = reqs_[running_[i]];
            const int remaining = (int)r.tokens.size() - r.computed;
            if (remaining != 1 || r.computed == 0) {
                ++i;
                continue;
            }
            if (cache_->extend(r.slot, r.computed + 1)) {
                push(r, 1);
                ++i;
                continue;
            }
            if (running_.size() == 1) {
                finish(r, FINISH_ABORT);  // alone and still no page: the pool cannot hold it
                break;
            }
            const bool self = running_.back() == r.id;
            preempt_newest();
            preempted = true;
            if (self) break;  // it was the newest itself; nothing after it
        }
        // 2. prompt portions of running requests, oldest first
        for (size_t i = 0; i < running_.size() && budget > 0; ++i) {
            Request& r = reqs_[running_[i]];
            const int remaining = (int)r.tokens.size() - r.computed;
            if (remaining == 1 && r.computed > 0) continue;  // handled above
            int n = std::min(std::min(remaining, cfg_.prefill_chunk_size), budget);
            n = fit_tokens(*cache_, r.slot, r.computed, n);
            if (n <= 0) continue;
            cache_->extend(r.slot, r.computed + n);
            push(r, n);
        }
        // 3. admit waiting requests in arrival order while slots, budget and pages last
        while (!preempted && !waiting_.empty() && budget > 0 && (int)running_.size() < cfg_.max_num_seqs) {
            Request& r = reqs_[waiting_.front()];
            const int slot = cache_->open_request();
            if (slot < 0) break;
            int n = std::min(std::min((int)r.tokens.size(), cfg_.prefill_chunk_size), budget);
            n = fit_tokens(*cache_, slot, 0, n);
            if (n <= 0) {
                cache_->close_request(slot);
                break;
            }
            r.slot = slot;
            r.computed = 0;
            cache_->extend(slot, n);
            waiting_.pop_front();
            running_.push_back(r.id);
            push(r, n);
        }
        if (!entries.empty() || running_.empty()) break;
        // running requests hold pages but none can move: take the newest one's pages
        if (running_.size() == 1) {
            finish(reqs_[running_[0]], FINISH_ABORT);
            continue;
        }
        preempt_newest();
    }
    return entries;
}

bool Scheduler::is_stop(const Request& r, int32_t tok) const {
    if (!r.ignore_eos && std::find(cfg_.eos_token_ids.begin(), cfg_.eos_token_ids.end(), tok) != cfg_.eos_token_ids.end())
        return true;
    // a stop sequence is hit when the generated tokens, with this one, end with it; the token itself then
    // stays out, what was generated before it stays (src/core/scheduler.rs:1459-1491, 617-647)
    const int generated = (int)r.tokens.size() - r.prompt_len;
    for (const std::vector<int32_t>& stop : r.stop_seqs) {
        const int before = (int)stop.size() - 1;
        if (stop.back() != tok || before > generated) continue;
        if (std::equal(stop.begin(), stop.end() - 1, r.tokens.end() - before)) return true;
    }
    return false;
}

std::vector<int64_t> Scheduler::drain_finished() {
    std::vector<int64_t> out;
    out.swap(finished_);
    return out;
}

void Scheduler::commit(const std::vector<StepEntry>& entries, const std::vector<int32_t>& sampled) {
    size_t k = 0;
    for (const StepEntry& e : entries) {
        auto it = reqs_.find(e.req_id);
        if (it == reqs_.end()) {  // ended and released while this step ran
            if (e.want) ++k;
            continue;
        }
        Request& r = it->second;
        if (r.finish != NOT_FINISHED || r.slot != e.slot) {  // ended or aborted meanwhile
            if (e.want) ++k;
            continue;
        }
        r.computed = e.start + e.count;
        cache_->advance(r.slot, r.computed);
        if (!e.want) continue;
        const int32_t tok = k < sampled.size() ? sampled[k] : -1;
        ++k;
        // the reference tests a sampled token before appending it: a stop or EOS token ends the
        // request and stays out of its output (src/core/scheduler.rs:617-647)
        if (is_stop(r, tok)) {
            r.hit_stop_token = true;
            finish(r, FINISH_STOP);
            continue;
        }
        r.tokens.push_back(tok);
        const int generated = (int)r.tokens.size() - r.prompt_len;
        if (generated >= r.max_tokens || (int)r.tokens.size() >= cfg_.max_model_len) {
            finish(r, FINISH_LENGTH);
        }
    }
}

std::vector<StepEntry> Scheduler::schedule_ahead(const std::vector<StepEntry>& prev, std::vector<int>* src) {
    std::vector<StepEntry> out;
    src->clear();
    if (!waiting_.empty() || prev.empty() || prev.size() != running_.size()) return out;
    int k = 0;
    for (const StepEntry& e : prev) {
        const int mine = e.want ? k++ : -1;
        auto it = reqs_.find(e.req_id);
        if (it == reqs_.end()) return {};
        const Request& r = it->second;
        if (r.finish != NOT_FINISHED || r.slot != e.slot || e.count != 1 || !e.want ||
            e.start + 1 != (int)r.tokens.size())
            return {};
        const int total = (int)r.tokens.size() + 1;   // what the request holds once prev is committed
        if (total - r.prompt_len >= r.max_tokens || total >= cfg_.max_model_len) continue;  // prev ends it
        StepEntry a;
        a.req_id = r.id;
        a.slot = r.slot;
        a.start = e.start + 1;
        a.count = 1;
        a.want = true;
        out.push_back(a);
        src->push_back(mine);
    }
    for (const StepEntry& a : out) {
        if (!cache_->extend(a.slot, a.start + 1)) {
            src->clear();
            return {};
        }
    }
    return out;
}

int Scheduler::finish_reason(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -1 : it->second.finish;
}
int Scheduler::output_length(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -1 : (int)it->second.tokens.size() - it->second.prompt_len;
}
int Scheduler::copy_output(int64_t id, int32_t* out, int capacity) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -1;
    const Request& r = it->second;
    const int n = std::min((int)r.tokens.size() - r.prompt_len, capacity);
    std::copy(r.tokens.begin() + r.prompt_len, r.tokens.begin() + r.prompt_len + n, out);
    return n;
}
int Scheduler::prompt_length(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -1 : it->second.prompt_len;
}
int Scheduler::num_drawn(int64_t id) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -1;
    const Request& r = it->second;
    return (int)r.tokens.size() - r.prompt_len + (r.hit_stop_token ? 1 : 0);
}
int Scheduler::copy_tail(int64_t id, int32_t* out, int n) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -1;
    const Request& r = it->second;
    n = std::min(n, (int)r.tokens.size());
    std::copy(r.tokens.end() - n, r.tokens.end(), out);
    return n;
}
bool Scheduler::release(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end() || it->second.finish == NOT_FINISHED) return false;
    reqs_.erase(it);
    return true;
}

}  // namespace xb
