// Continuous batching on the host: admission, cutting prompts into portions under a token budget,
// decoding, finishing, freeing, and what happens when pages run out.
//
// The reference alternates prefill-only and decode-only steps (src/core/scheduler.rs:236-408),
// re-queues a sequence after every prompt chunk (:842-864), and under page pressure evicts, swaps
// to the CPU or drops the oldest request (:346-372, src/core/engine.rs:1604-1621).  Here one step
// mixes single decode tokens with prompt portions; when a decode cannot get its page the newest
// running request is preempted: its pages go back, and it waits at the head of the queue with its
// generated tokens as part of its prompt (recomputed on re-admission).  Nothing is swapped.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <string>
#include <vector>

#include "cache_manager.h"

namespace xb {

struct SchedulerConfig {
    int max_num_seqs = 32;
    int max_num_batched_tokens = 8192;
    int prefill_chunk_size = 8192;
    int max_model_len = 1 << 30;
    std::vector<int32_t> eos_token_ids;
};

enum FinishReason : int { NOT_FINISHED = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_ABORT = 3 };

enum AddStatus : int {
    ADD_OK = 0,
    ADD_EMPTY_PROMPT = 1,
    ADD_TOO_LONG = 2,      // prompt does not leave room for one token under max_model_len
    ADD_NEVER_FITS = 3,    // prompt + max_tokens needs more pages than a pool has
    ADD_DUPLICATE = 4,
};

struct StepEntry {
    int64_t req_id;
    int slot;
    int start;   // tokens already in the cache
    int count;   // tokens this step runs
    bool want;   // the portion ends the known tokens: logits at its last token are wanted
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, const SchedulerConfig& cfg);

    // `stop_ids` holds the request's stop sequences back to back, `stop_lens` the length of each
    // (n_stop of them): a sequence of one token stops on that token; a longer one stops when the
    // generated tokens end with it (src/core/scheduler.rs:1459-1491).
    AddStatus add(int64_t req_id, const int32_t* prompt, int n, int max_tokens, bool ignore_eos,
                  const int32_t* stop_ids, const int32_t* stop_lens, int n_stop);
    bool abort(int64_t req_id);

    // Decide the next step.  Pages for every entry are taken here.  `tokens` receives the entries'
    // token ids back to back.  Returns the entries (empty when nothing can run).
    std::vector<StepEntry> schedule(std::vector<int32_t>* tokens);
    // The step ran.  `sampled` holds one token per entry with want == true, in entry order.
    void commit(const std::vector<StepEntry>& entries, const std::vector<int32_t>& sampled);
    // The step after `prev`, decided while `prev` still runs (its tokens are not known yet): possible
    // when nothing waits and `prev` decodes one token for every running request.  Each entry decodes
    // the token that `prev` will sample for its request; `src` receives, per entry, the index of that
    // token among prev's sampled tokens.  Requests that `prev` ends by length are left out; one that
    // ends on a stop token is found out at commit, and its entry of this step is then ignored.
    // Pages are taken here.  Empty when the step cannot be decided ahead (then nothing has changed
    // but pages reserved for requests that will need them anyway).
    std::vector<StepEntry> schedule_ahead(const std::vector<StepEntry>& prev, std::vector<int>* src);
    // Ids that finished (or were aborted) since the last call, in the order they ended.
    std::vector<int64_t> drain_finished();

    int num_waiting() const { return (int)waiting_.size(); }
    int num_running() const { return (int)running_.size(); }
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int preemptions() const { return preemptions_; }

    // Finished requests stay readable until released.
    int finish_reason(int64_t req_id) const;
    int output_length(int64_t req_id) const;
    int copy_output(int64_t req_id, int32_t* out, int capacity) const;
    int prompt_length(int64_t req_id) const;
    int num_drawn(int64_t req_id) const;   // tokens sampled so far (the sampler's counter)
    int copy_tail(int64_t req_id, int32_t* out, int n) const;  // last n known tokens
    bool release(int64_t req_id);

private:
    struct Request {
        int64_t id = 0;
        std::vector<int32_t> tokens;  // prompt, then generated
        int prompt_len = 0;
        int computed = 0;             // tokens whose keys/values are cached
        int slot = -1;
        int max_tokens = 0;
        bool ignore_eos = false;
        std::vector<std::vector<int32_t>> stop_seqs;
        int finish = NOT_FINISHED;
        bool hit_stop_token = false;
    };
    bool is_stop(const Request& r, int32_t tok) const;
    void preempt_newest();
    void finish(Request& r, int reason);

    CacheManager* cache_;
    SchedulerConfig cfg_;
    std::map<int64_t, Request> reqs_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;   // admission order, oldest first
    int preemptions_ = 0;
    std::vector<int64_t> finished_;
};

}  // namespace xb
