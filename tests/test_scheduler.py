"""The scheduler's decisions, with a fake step that makes up tokens (no GPU)."""
import random

import pytest

from xinfer_b200.cache import CacheGroup, CacheManager
from xinfer_b200.engine.scheduler import Scheduler, SchedulerError


def make(pages=64, page=16, seqs=4, budget=64, chunk=32, max_len=512, eos=(), window=None):
    cm = CacheManager([CacheGroup(page, pages, window)], max_requests=seqs)
    return cm, Scheduler(cm, max_num_seqs=seqs, max_num_batched_tokens=budget, prefill_chunk_size=chunk,
                         max_model_len=max_len, eos_token_ids=eos)


def run(sched, token_of=lambda e, step: 7, max_steps=10_000):
    """Drive to completion; returns (list of batches, {id: finish step})."""
    batches, ended = [], {}
    for step in range(max_steps):
        if not sched.has_work():
            break
        entries = sched.schedule()
        for i in sched.drain_finished():
            ended[i] = step
        if not entries:
            continue
        batches.append(entries)
        for i in sched.commit([token_of(e, step) for e in entries if e.want]):
            ended[i] = step
    assert not sched.has_work()
    return batches, ended


def test_prompt_is_cut_under_chunk_and_budget_then_decoded():
    cm, s = make(budget=40, chunk=32)
    s.add(0, list(range(100)), max_tokens=3)
    batches, ended = run(s)
    sizes = [len(b[0].tokens) for b in batches]
    assert sizes == [32, 32, 32, 4, 1, 1]
    assert [b[0].start for b in batches] == [0, 32, 64, 96, 100, 101]
    assert [b[0].want for b in batches] == [False, False, False, True, True, True]
    assert batches[0][0].tokens.tolist() == list(range(32))
    assert s.output(0) == [7, 7, 7] and s.finish_reason(0) == "length"
    assert cm.live_requests() == 0 and cm.free_pages() == 64
    s.release(0)


def test_decodes_come_first_and_share_a_step_with_prompt_portions():
    cm, s = make(budget=24, chunk=16)
    s.add(0, [1] * 10, max_tokens=8)
    e = s.schedule()
    assert [(x.req_id, len(x.tokens), x.want) for x in e] == [(0, 10, True)]
    s.commit([9])
    s.add(1, [2] * 40, max_tokens=2)
    e = s.schedule()
    # one decode token of request 0, then a portion of request 1 cut by the chunk size
    assert [(x.req_id, len(x.tokens), x.start, x.want) for x in e] == [(0, 1, 10, True), (1, 16, 0, False)]
    s.commit([9])
    e = s.schedule()
    assert [(x.req_id, len(x.tokens), x.start) for x in e] == [(0, 1, 11), (1, 16, 16)]
    s.commit([9])
    e = s.schedule()
    assert [(x.req_id, len(x.tokens), x.start, x.want) for x in e] == [(0, 1, 12, True), (1, 8, 32, True)]
    total = sum(len(x.tokens) for x in e)
    assert total <= 24


def test_token_budget_cuts_a_portion_down():
    cm, s = make(budget=20, chunk=16, seqs=4)
    for i in range(3):
        s.add(i, [i] * 12, max_tokens=1)
    e = s.schedule()
    assert [(x.req_id, len(x.tokens)) for x in e] == [(0, 12), (1, 8)]
    s.commit([5])   # request 0 finishes (max_tokens 1)
    e = s.schedule()
    assert [(x.req_id, len(x.tokens), x.start) for x in e] == [(1, 4, 8), (2, 12, 0)]


def test_max_num_seqs_limits_admission():
    cm, s = make(seqs=2, budget=64)
    for i in range(4):
        s.add(i, [1, 2, 3], max_tokens=2)
    e = s.schedule()
    assert [x.req_id for x in e] == [0, 1] and s.num_waiting == 2
    _, ended = run(s)
    assert sorted(ended) == [0, 1, 2, 3]


def test_finish_rules():
    cm, s = make(eos=(99,), max_len=12)
    s.add(0, [1, 2, 3], max_tokens=50)                          # ends on EOS, which stays out
    s.add(1, [1, 2, 3], max_tokens=50, ignore_eos=True)         # ignores EOS, ends at max_model_len
    s.add(2, [1, 2, 3], max_tokens=50, stop_token_ids=[42])     # ends on its own stop token
    s.add(3, [1, 2, 3], max_tokens=2)

    def tok(e, step):
        if e.req_id == 0:
            return 99 if step == 2 else 5
        if e.req_id == 2:
            return 42 if step == 1 else 5
        return 99 if e.req_id == 1 else 5
    run(s, tok)
    assert s.output(0) == [5, 5] and s.finish_reason(0) == "stop"
    assert s.finish_reason(1) == "length" and len(s.output(1)) == 9 and s.prompt_length(1) == 3
    assert s.output(2) == [5] and s.finish_reason(2) == "stop"
    assert s.output(3) == [5, 5] and s.finish_reason(3) == "length"
    assert s.num_drawn(0) == 3 and s.num_drawn(3) == 2
    assert cm.free_pages() == 64


def test_add_errors():
    cm, s = make(pages=4, page=16, max_len=128)
    with pytest.raises(SchedulerError, match="empty"):
        s.add(0, [], 4)
    with pytest.raises(SchedulerError, match="too long"):
        s.add(0, [1] * 128, 4)
    with pytest.raises(SchedulerError, match="never fit"):
        s.add(0, [1] * 60, 10)       # 70 tokens need 5 pages, the pool has 4
    s.add(0, [1] * 50, 10)
    with pytest.raises(SchedulerError, match="exists"):
        s.add(0, [1], 1)


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    # 6 pages of 4 tokens: two requests of 8 prompt tokens fit, but not both growing to 14
    cm, s = make(pages=6, page=4, seqs=2, budget=64, chunk=64, max_len=64)
    s.add(0, list(range(10, 18)), max_tokens=6)
    s.add(1, list(range(20, 28)), max_tokens=6)
    log = []

    def tok(e, step):
        log.append((step, e.req_id, e.start, len(e.tokens)))
        return 100 + e.req_id
    batches, ended = run(s, tok)
    assert s.preemptions >= 1
    assert s.output(0) == [100] * 6 and s.output(1) == [101] * 6
    assert ended[0] < ended[1]                       # the older request was never disturbed
    # the preempted request came back with its prompt and generated tokens as one portion from 0
    redo = [b for b in batches for e in b if e.req_id == 1 and e.start == 0]
    assert len(redo) == 2
    again = [e for e in redo[1] if e.req_id == 1][0]
    assert again.tokens.tolist()[:8] == list(range(20, 28)) and set(again.tokens.tolist()[8:]) == {101}
    assert cm.free_pages() == 6 and cm.live_requests() == 0
    cm.check_consistent()


def test_a_request_alone_that_cannot_grow_is_aborted_not_spun_on():
    cm, s = make(pages=2, page=4, seqs=1, budget=64, chunk=64, max_len=64)
    s.add(0, [1] * 6, max_tokens=2)     # fits: 8 tokens = 2 pages
    run(s)
    assert s.finish_reason(0) == "length"
    # a second pool user that takes a page away makes the lone request impossible to grow
    cm2, s2 = make(pages=3, page=4, seqs=2, budget=64, chunk=64, max_len=64)
    other = cm2.open_request()
    assert cm2.extend(other, 4)
    s2.add(0, [1] * 8, max_tokens=4)
    _, ended = run(s2)
    assert s2.finish_reason(0) == "abort" and cm2.free_pages() == 2


def test_abort_frees_pages():
    cm, s = make()
    s.add(0, [1] * 30, max_tokens=5)
    s.schedule()
    s.commit([])
    assert cm.free_pages() < 64
    assert s.abort(0) and not s.abort(0)
    assert cm.free_pages() == 64 and s.finish_reason(0) == "abort" and s.drain_finished() == [0]


def test_abort_of_a_waiting_request_and_of_one_whose_step_is_not_recorded_yet():
    cm, s = make(seqs=1)
    s.add(0, [1] * 10, max_tokens=4)
    s.add(1, [2] * 10, max_tokens=4)          # waits: one request slot
    assert s.abort(1) and s.finish_reason(1) == "abort" and s.drain_finished() == [1] and s.output(1) == []
    entries = s.schedule()                     # request 0's prompt, scheduled ...
    assert [e.req_id for e in entries] == [0]
    assert s.abort(0) and cm.free_pages() == 64   # ... and aborted before its token is recorded
    assert s.commit([9]) == [0] and s.output(0) == []   # reported as ended; the token of a request that is gone is dropped
    assert s.drain_finished() == [] and not s.has_work()
    cm.check_consistent()
    s.add(2, [3] * 5, max_tokens=2)            # the scheduler goes on
    batches, ended = run(s)
    assert s.output(2) == [7, 7] and cm.free_pages() == 64


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_and_leave_the_pool_whole(seed):
    rng = random.Random(seed)
    page = rng.choice([4, 8, 16])
    pages = rng.randint(12, 40)
    window = rng.choice([None, None, 9, 23])
    cm, s = make(pages=pages, page=page, seqs=rng.randint(2, 5), budget=rng.randint(8, 48),
                 chunk=rng.randint(4, 32), max_len=200, eos=(1,), window=window)
    want = {}
    nxt = 0
    for step in range(3000):
        if nxt < 25 and rng.random() < 0.3:
            n, m = rng.randint(1, 60), rng.randint(1, 30)
            try:
                s.add(nxt, [rng.randint(2, 50) for _ in range(n)], m)
                want[nxt] = (n, m)
            except SchedulerError:
                pass
            nxt += 1
        if not s.has_work():
            if nxt >= 25:
                break
            continue
        entries = s.schedule()
        s.drain_finished()
        total = sum(len(e.tokens) for e in entries)
        assert len({e.req_id for e in entries}) == len(entries)
        for e in entries:
            assert cm.length(e.slot) == e.start
            assert len(cm.table(e.slot)) * page >= e.start + len(e.tokens)
        s.commit([rng.choice([1, 7, 8, 9]) if rng.random() < 0.05 else 7 for e in entries if e.want])
        cm.check_consistent()
    assert not s.has_work()
    for i, (n, m) in want.items():
        assert s.finish_reason(i) in ("stop", "length")
        assert len(s.output(i)) <= m
    assert cm.free_pages() == pages and cm.live_requests() == 0


# ---- deciding the next step while the current one runs ------------------------------------------------
def run_ahead(sched, token_of, max_steps=10_000):
    """Drive to completion the way the engine does: while a step "runs", the next is decided from
    it; its tokens are made up from what the running step will have sampled."""
    flights, ended, outputs = [], {}, {}
    flight = None
    for step in range(max_steps):
        if flight is None:
            if not sched.has_work():
                break
            entries = sched.schedule()
            for i in sched.drain_finished():
                ended[i] = step
            if not entries:
                continue
            flight = (entries, False)
        entries, was_ahead = flight
        flights.append(flight)
        nxt = sched.schedule_ahead() if all(e.want and len(e.tokens) == 1 for e in entries) else []
        sampled = [token_of(e, step) for e in entries if e.want]
        for i in sched.commit(sampled):
            ended[i] = step
            outputs[i] = sched.output(i)
            sched.release(i)
        flight = (nxt, True) if nxt else None
        if flight is not None and all(e.req_id in ended for e in nxt):
            sched.commit([0] * len(nxt))
            flight = None
    assert not sched.has_work()
    return flights, ended, outputs


def test_a_decode_step_is_decided_while_the_one_before_runs():
    cm, s = make(budget=64, chunk=32)
    s.add(0, [1] * 5, max_tokens=6)
    s.add(1, [2] * 9, max_tokens=4)
    assert s.schedule_ahead() == []                       # nothing runs yet
    e = s.schedule()
    assert [len(x.tokens) for x in e] == [5, 9]
    assert s.schedule_ahead() == []                       # the running step is a prompt step
    s.commit([11, 12])
    e = s.schedule()
    assert [(x.req_id, x.start, len(x.tokens)) for x in e] == [(0, 5, 1), (1, 9, 1)]
    a = s.schedule_ahead()
    assert [(x.req_id, x.slot, x.start, x.src, x.want) for x in a] == [(0, e[0].slot, 6, 0, True), (1, e[1].slot, 10, 1, True)]
    assert s.schedule_ahead() == []                       # only one step ahead
    s.commit([21, 22])                                    # the running step's tokens arrive
    a2 = s.schedule_ahead()                               # ... and the step after the one decided ahead
    assert [(x.req_id, x.start) for x in a2] == [(0, 7), (1, 11)]
    s.commit([31, 32])
    # request 1 has 3 of its 4 tokens: the step in flight gives the fourth and ends it by length
    a3 = s.schedule_ahead()
    assert [(x.req_id, x.start, x.src) for x in a3] == [(0, 8, 0)]
    assert s.commit([41, 42]) == [1]
    assert s.output(1) == [12, 22, 32, 42] and s.finish_reason(1) == "length"
    assert s.commit([51]) == []
    assert s.output(0) == [11, 21, 31, 41, 51]


def test_a_stop_token_found_late_drops_the_token_computed_in_vain():
    cm, s = make(eos=(99,))
    s.add(0, [1] * 4, max_tokens=50)
    s.add(1, [2] * 4, max_tokens=50)
    s.schedule(); s.commit([5, 6])
    s.schedule()
    a = s.schedule_ahead()
    assert [x.req_id for x in a] == [0, 1]
    assert s.commit([99, 7]) == [0]                       # request 0 stops; its entry of the next step is void
    s.release(0)
    assert s.commit([1234, 8]) == []                      # the void entry's token is skipped, request 1 gets its own
    assert s.output(1) == [6, 7, 8]
    assert cm.live_requests() == 1
    # the step after: only request 1 is left
    e = s.schedule()
    assert [(x.req_id, x.start) for x in e] == [(1, 6)]


def test_nothing_is_decided_ahead_when_requests_wait_or_pages_are_short():
    cm, s = make(seqs=1)
    s.add(0, [1] * 4, max_tokens=9)
    s.add(1, [2] * 4, max_tokens=9)                       # waits for the only slot
    s.schedule(); s.commit([5])
    s.schedule()
    assert s.schedule_ahead() == []
    s.commit([5])
    cm2, s2 = make(pages=4, page=4, seqs=2)
    s2.add(0, [1] * 7, max_tokens=3)
    s2.add(1, [2] * 7, max_tokens=3)
    s2.schedule(); s2.commit([5, 5])                      # 8 tokens known each, 7 cached: all four pages in use
    e = s2.schedule()
    assert [(x.start, len(x.tokens)) for x in e] == [(7, 1), (7, 1)]
    assert s2.schedule_ahead() == []                      # the tokens after these would need a fifth page


@pytest.mark.parametrize("seed", range(6))
def test_deciding_ahead_gives_the_same_outputs(seed):
    rng = random.Random(seed)
    reqs = [(i, [rng.randrange(50) for _ in range(rng.randrange(1, 40))], rng.randrange(1, 25)) for i in range(7)]

    def tok(e, step):   # a token that depends only on the request and its position: 3 is the stop token
        return (e.req_id * 7 + (e.start + len(e.tokens)) * 13) % 17

    outs = []
    for ahead in (False, True):
        cm, s = make(pages=40, page=4, seqs=4, budget=48, chunk=16, eos=(3,))
        for i, p, m in reqs:
            s.add(i, p, max_tokens=m)
        if ahead:
            flights, ended, outputs = run_ahead(s, tok)
            assert any(was for _, was in flights), "some steps must have been decided ahead"
        else:
            outputs = {}
            _, ended = run(s, tok)
            for i in ended:
                outputs[i] = s.output(i)
        assert cm.live_requests() == 0 and cm.free_pages() == 40
        cm.check_consistent()
        outs.append(outputs)
    assert outs[0] == outs[1]


def test_a_failed_step_aborts_what_was_scheduled_and_nothing_else():
    """A step fails with one batch running and one decided ahead: the requests of both end as aborted,
    their pages go back, nothing stays scheduled; a request that only waited is served afterwards."""
    cm, s = make(pages=16, page=4, seqs=2)
    s.add(0, [1] * 5, max_tokens=9)
    s.add(1, [2] * 6, max_tokens=9)
    s.add(2, [3] * 4, max_tokens=2)                          # waits: both slots are taken
    s.schedule(); s.commit([5, 5])                           # prompts done, first tokens known
    running = s.schedule()
    assert [e.req_id for e in running] == [0, 1] and s.schedule_ahead() == []     # request 2 waits: nothing ahead
    assert sorted(s.fail_steps()) == [0, 1]
    assert s.finish_reason(0) == s.finish_reason(1) == "abort"
    assert s.output(0) == [5] and s.output(1) == [5]         # what was recorded before stays readable
    assert cm.live_requests() == 0 and cm.free_pages() == 16
    cm.check_consistent()
    assert s.fail_steps() == []                              # nothing is scheduled any more
    s.release(0); s.release(1)
    batches, ended = run(s)
    assert list(ended) == [2] and s.finish_reason(2) == "length" and len(s.output(2)) == 2
    assert cm.free_pages() == 16

    # with a step decided ahead: both steps' requests go
    cm, s = make(pages=16, page=4, seqs=2)
    s.add(0, [1] * 5, max_tokens=9)
    s.add(1, [2] * 6, max_tokens=9)
    s.schedule(); s.commit([5, 5])
    s.schedule()
    ahead = s.schedule_ahead()
    assert [e.req_id for e in ahead] == [0, 1]
    assert sorted(s.fail_steps()) == [0, 1] and not s.has_work()
    assert cm.live_requests() == 0 and cm.free_pages() == 16
    cm.check_consistent()
    s.add(7, [4] * 3, max_tokens=2)                          # the scheduler goes on
    _, ended = run(s)
    assert list(ended) == [7]


def test_stop_sequences_of_several_tokens():
    """A stop sequence ends a request when the generated tokens end with it; its last token stays out, what
    came before stays in; the prompt does not count; single ids and sequences mix."""
    toks = [4, 9, 9, 2, 7, 9, 2, 5, 1]

    def feed(stops, prompt=(9, 2), max_tokens=9):
        cm, s = make()
        s.add(0, list(prompt), max_tokens=max_tokens, stop_token_ids=stops)
        i = [0]

        def tok(e, step):
            i[0] += 1
            return toks[i[0] - 1]
        run(s, tok)
        return s.output(0), s.finish_reason(0)

    assert feed([[9, 2]]) == ([4, 9, 9], "stop")                 # generated ... 9 then 2: stops, 2 stays out
    assert feed([[9, 2, 5]]) == ([4, 9, 9, 2, 7, 9, 2], "stop")  # the first 9 2 is followed by 7: no match; the second by 5
    assert feed([[2, 4]]) == (toks, "length")                    # the prompt's 2 does not count
    assert feed([7, [9, 9, 9]]) == ([4, 9, 9, 2], "stop")        # a single id beside a sequence that never comes
    assert feed([[4]]) == ([], "stop")                           # a sequence of one is a stop token
    assert feed([[1, 1], []]) == (toks, "length")                # never hit; an empty sequence is nothing
