"""Python face of the native scheduler (csrc/host/scheduler.cpp): admission, prompt portions under
a token budget, decoding, finishing, freeing, preemption when pages run out."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from ..cache.manager import CacheManager
from ..native import host_lib

FINISH_REASONS = {0: None, 1: "stop", 2: "length", 3: "abort"}
_ADD_ERRORS = {
    1: "the prompt is empty",
    2: "the prompt is too long: it must leave room for at least one token under max_model_len",
    3: "the request can never fit: prompt + max_tokens needs more pages than the cache pool has",
    4: "a request with this id exists already",
}


class SchedulerError(RuntimeError):
    pass


@dataclass
class ScheduledEntry:
    req_id: int
    slot: int
    start: int     # tokens already cached
    tokens: np.ndarray
    want: bool     # logits at the last token are wanted (the portion ends the known tokens)
    # for a step decided ahead: which of the running step's sampled tokens this entry decodes
    src: Optional[int] = None


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk_size: int, max_model_len: int, eos_token_ids: Sequence[int] = ()):
        self._lib = host_lib()
        self.cache = cache
        eos = np.asarray(list(eos_token_ids), dtype=np.int32)
        self._h = self._lib.xb_sched_create(cache.handle, int(max_num_seqs), int(max_num_batched_tokens),
                                            int(prefill_chunk_size), int(max_model_len),
                                            eos.ctypes.data if len(eos) else None, len(eos))
        if not self._h:
            raise SchedulerError("invalid scheduler options (all sizes must be positive, max_model_len > 1)")
        self._cap_e = int(max_num_seqs) + 8
        self._cap_t = int(max_num_batched_tokens) + 8
        self._ids = np.zeros(self._cap_e, dtype=np.int64)
        self._slots = np.zeros(self._cap_e, dtype=np.int32)
        self._starts = np.zeros(self._cap_e, dtype=np.int32)
        self._counts = np.zeros(self._cap_e, dtype=np.int32)
        self._wants = np.zeros(self._cap_e, dtype=np.int32)
        self._tokens = np.zeros(self._cap_t, dtype=np.int32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.xb_sched_destroy(h)

    def add(self, req_id: int, prompt: Sequence[int], max_tokens: int, ignore_eos: bool = False,
            stop_token_ids: Sequence = ()) -> None:
        """``stop_token_ids``: token ids and / or sequences of token ids.  A single id ends the request
        when it is sampled; a sequence ends it when the generated tokens end with it.  The token that
        completes a stop stays out of the output (src/core/scheduler.rs:1459-1491, 617-647)."""
        p = np.asarray(list(prompt), dtype=np.int32)
        seqs = [[int(s)] if isinstance(s, (int, np.integer)) else [int(t) for t in s] for s in stop_token_ids]
        seqs = [q for q in seqs if q]
        flat = np.asarray([t for q in seqs for t in q], dtype=np.int32)
        lens = np.asarray([len(q) for q in seqs], dtype=np.int32)
        rc = self._lib.xb_sched_add(self._h, int(req_id), p.ctypes.data if len(p) else None, len(p), int(max_tokens),
                                    int(bool(ignore_eos)), flat.ctypes.data if len(flat) else None,
                                    lens.ctypes.data if len(lens) else None, len(lens))
        if rc:
            raise SchedulerError(_ADD_ERRORS.get(rc, f"add failed ({rc})"))

    def abort(self, req_id: int) -> bool:
        return bool(self._lib.xb_sched_abort(self._h, int(req_id)))

    def schedule(self) -> List[ScheduledEntry]:
        n_tok = ctypes.c_int(0)
        n = self._lib.xb_sched_schedule(self._h, self._cap_e, self._ids.ctypes.data, self._slots.ctypes.data,
                                        self._starts.ctypes.data, self._counts.ctypes.data, self._wants.ctypes.data,
                                        self._cap_t, self._tokens.ctypes.data, ctypes.byref(n_tok))
        if n < 0:
            raise SchedulerError("the scheduled batch exceeds the scheduler's buffers")
        out, t = [], 0
        for i in range(n):
            c = int(self._counts[i])
            out.append(ScheduledEntry(int(self._ids[i]), int(self._slots[i]), int(self._starts[i]),
                                      self._tokens[t:t + c].copy(), bool(self._wants[i])))
            t += c
        return out

    def schedule_ahead(self) -> List[ScheduledEntry]:
        """The step after the one that was scheduled and still runs, decided before its tokens are
        known: one decode token per running request (``tokens`` is a placeholder; ``src`` says
        which sampled token of the running step takes its place).  Empty when that cannot be done:
        something waits, the running step is not all decode, pages are short.  A request that the
        running step ends on a stop token still gets an entry; commit ignores it."""
        src = np.zeros(self._cap_e, dtype=np.int32)
        n = self._lib.xb_sched_schedule_ahead(self._h, self._cap_e, self._ids.ctypes.data, self._slots.ctypes.data,
                                              self._starts.ctypes.data, src.ctypes.data)
        if n < 0:
            raise SchedulerError("the scheduled batch exceeds the scheduler's buffers")
        return [ScheduledEntry(int(self._ids[i]), int(self._slots[i]), int(self._starts[i]),
                               np.zeros(1, dtype=np.int32), True, int(src[i])) for i in range(n)]

    def commit(self, sampled: Sequence[int]) -> List[int]:
        """Record the oldest scheduled step that is not yet recorded; ``sampled`` holds one token per
        entry that wanted logits, in entry order.  Returns the ids that ended (finished or aborted)."""
        s = np.asarray(list(sampled), dtype=np.int32)
        self._lib.xb_sched_commit(self._h, s.ctypes.data if len(s) else None, len(s))
        return self.drain_finished()

    def fail_steps(self) -> List[int]:
        """A scheduled step failed: abort every request of the steps that are scheduled and not
        recorded (the running one and the one decided ahead), give their pages back and leave nothing
        scheduled.  Returns the ids that ended."""
        self._lib.xb_sched_fail_steps(self._h)
        return self.drain_finished()

    def drain_finished(self) -> List[int]:
        buf = np.zeros(max(self._cap_e, 64), dtype=np.int64)
        out: List[int] = []
        while True:
            n = self._lib.xb_sched_drain_finished(self._h, buf.ctypes.data, len(buf))
            out += [int(x) for x in buf[:n]]
            if n < len(buf):
                return out

    @property
    def num_waiting(self) -> int:
        return self._lib.xb_sched_num_waiting(self._h)

    @property
    def num_running(self) -> int:
        return self._lib.xb_sched_num_running(self._h)

    @property
    def preemptions(self) -> int:
        return self._lib.xb_sched_preemptions(self._h)

    def has_work(self) -> bool:
        return self.num_waiting + self.num_running > 0

    def finish_reason(self, req_id: int) -> Optional[str]:
        return FINISH_REASONS.get(self._lib.xb_sched_finish_reason(self._h, int(req_id)))

    def prompt_length(self, req_id: int) -> int:
        return self._lib.xb_sched_prompt_length(self._h, int(req_id))

    def num_drawn(self, req_id: int) -> int:
        return self._lib.xb_sched_num_drawn(self._h, int(req_id))

    def output(self, req_id: int) -> List[int]:
        n = self._lib.xb_sched_output_length(self._h, int(req_id))
        if n < 0:
            raise SchedulerError(f"unknown request {req_id}")
        buf = np.zeros(max(n, 1), dtype=np.int32)
        self._lib.xb_sched_copy_output(self._h, int(req_id), buf.ctypes.data, n)
        return buf[:n].tolist()

    def tail(self, req_id: int, n: int) -> List[int]:
        buf = np.zeros(max(n, 1), dtype=np.int32)
        got = self._lib.xb_sched_copy_tail(self._h, int(req_id), buf.ctypes.data, n)
        return buf[:max(got, 0)].tolist()

    def release(self, req_id: int) -> None:
        self._lib.xb_sched_release(self._h, int(req_id))
