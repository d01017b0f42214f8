"""The Python entry point, in the manner of the reference's package (xinfer.pyi:191-238,
src/py/mod.rs:28-152): ``Engine(econfig, dtype)`` with ``generate_sync`` and ``generate_stream``.
Prompts are lists of token ids (the reference takes chat messages and tokenises them; templates
and tokenisers are outside this engine).

One loop iteration = schedule -> step -> sample -> commit, as the reference's
prepare_step / run_forward / finish_step (src/core/engine.rs:1034, 1085, 1363).

A step that fails (no pages at the last moment, an error word from a kernel, a bounded wait that
gave up, a launch error) ends the requests of the batches that were scheduled and not yet recorded
with ``finish_reason == "abort"`` and the reason in ``error``; their pages go back, nothing stays
scheduled, and the loop goes on with the other requests.  The reference cancels every request with
the reason and keeps its loop alive (src/core/engine.rs:2392-2408).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..config import EngineConfig
from ..config.generation import GenerationConfig, join_eos
from ..sampling import SamplingParams
from ..sampling.sampler import PENALTY_HISTORY, Sampler
from .runner import ModelRunner, StepError, StepInput
from .scheduler import Scheduler, SchedulerError


@dataclass
class GenerationOutput:
    """Fields as in the reference (src/core/mod.rs:13-30); ``decode_output`` holds token ids."""

    seq_id: int
    prompt_length: int
    prompt_start_time: int    # milliseconds since the epoch
    decode_start_time: int
    decode_finish_time: int
    decoded_length: int
    decode_output: List[int]
    finish_reason: Optional[str] = None
    # why the request was aborted, when a step it was part of failed
    error: Optional[str] = None


@dataclass
class StreamItem:
    """``datatype`` is "TOKEN_ID" (data: int), "DONE" (data: (seq_id, prompt_length,
    decoded_length, decode_ms)) or "ERROR" (data: str), after src/py/mod.rs:178-279."""

    datatype: str
    data: object


@dataclass
class _Live:
    params: SamplingParams
    seed: int
    prompt_len: int
    t_start: float
    t_first: float = 0.0


def _ms(t: float) -> int:
    return int(t * 1000)


@dataclass
class _Flight:
    """A batch that is queued on the device."""
    wanted: list
    tokens_dev: Optional[torch.Tensor] = None
    sampler: Optional[Sampler] = None
    penalties: bool = False


class EngineStream:
    """The iterator ``generate_stream`` returns, with the reference's attributes (xinfer.pyi: EngineStream):
    ``finished``, ``seq_id``, ``prompt_length``, ``cancelled`` and ``cancel()``.  Every ``next`` runs engine
    steps until the request has new tokens (or has ended) and hands them out one by one."""

    def __init__(self, engine: "Engine", seq_id: int, prompt_length: int):
        self.engine = engine
        self.seq_id = seq_id
        self.prompt_length = prompt_length
        self.finished = False
        self.cancelled = False
        self._queue: List[StreamItem] = []
        self._streamed = 0

    def cancel(self) -> None:
        if not self.finished:
            self.cancelled = self.engine.cancel(self.seq_id) or self.cancelled

    def __iter__(self) -> "EngineStream":
        return self

    def _pull(self) -> None:
        eng, seq_id = self.engine, self.seq_id
        if seq_id in eng._live:
            before = (eng.stats["steps"], len(eng._live))
            eng.step()
            if (eng.stats["steps"], len(eng._live)) == before and not eng.has_work() and seq_id in eng._live:
                eng.cancel(seq_id)     # nothing can move this request any further: end it instead of spinning
        done = eng._done.get(seq_id)
        src = done.decode_output if done is not None else eng.scheduler.output(seq_id)
        self._queue += [StreamItem("TOKEN_ID", int(t)) for t in src[self._streamed:]]
        self._streamed = len(src)
        if done is not None:
            eng._done.pop(seq_id)
            if done.error is not None:
                self._queue.append(StreamItem("ERROR", done.error))
            else:
                self._queue.append(StreamItem("DONE", (seq_id, done.prompt_length, done.decoded_length,
                                                       done.decode_finish_time - done.decode_start_time)))
            self.finished = True

    def __next__(self) -> StreamItem:
        while not self._queue:
            if self.finished:
                raise StopIteration
            self._pull()
        return self._queue.pop(0)


class Engine:
    def __init__(self, econfig: EngineConfig, dtype: str = "bf16", runner: Optional[ModelRunner] = None):
        """``runner``: a prepared model runner (for instance ``ModelRunner.random``) to use instead
        of loading ``econfig``'s model folder."""
        econfig.validate()
        self.econfig = econfig
        self.runner = runner if runner is not None else ModelRunner(
            econfig.model_dir(), dtype, block_size=econfig.block_size, num_blocks=econfig.num_blocks,
            max_num_seqs=econfig.max_num_seqs, kv_fraction=econfig.kv_fraction, device=econfig.device,
            max_model_len=econfig.max_model_len, poison_freed_pages=econfig.poison_freed_pages)
        self.max_model_len = self.runner.max_model_len
        # defaults for what a request leaves unset: the engine's own, then the model folder's generation_config.json
        folder = econfig.weight_path or econfig.model_id
        from_folder = GenerationConfig.load(folder) if folder and os.path.isdir(folder) else None
        self.generation_cfg = econfig.generation_cfg.over(from_folder) if econfig.generation_cfg is not None else from_folder
        self.eos_token_ids = join_eos(self.runner.plan.eos_token_ids, from_folder)
        budget = min(econfig.max_num_batched_tokens, max(self.runner.kv_cache_tokens(), 1))
        self.scheduler = Scheduler(
            self.runner.cache, max_num_seqs=econfig.max_num_seqs, max_num_batched_tokens=budget,
            prefill_chunk_size=econfig.prefill_chunk_size, max_model_len=self.max_model_len,
            eos_token_ids=self.eos_token_ids)
        # two sets of pinned buffers (two batches can be in flight); both leave their ids in the runner's
        # buffer, where the step after reads them on the device
        self.samplers = [Sampler(self.runner.device, econfig.max_num_seqs, out_dev=self.runner.sampled_tokens,
                                 err_word=self.runner.err) for _ in range(2)]
        self.sampler = self.samplers[0]
        self._sampler_i = 0
        self._flight: Optional[_Flight] = None    # a batch queued on the device whose tokens are not recorded yet
        self.run_ahead = not econfig.disable_run_ahead
        self.seed = 0 if econfig.seed is None else int(econfig.seed)
        self._next_id = 0
        self._live: Dict[int, _Live] = {}
        self._done: Dict[int, GenerationOutput] = {}
        self.use_graphs = not econfig.disable_cuda_graph
        # counters (the reference logs the same two throughputs, src/core/engine.rs:1584-1716)
        self.stats = {"steps": 0, "prompt_tokens": 0, "decoded_tokens": 0, "preemptions": 0, "steps_decided_ahead": 0,
                      "failed_steps": 0}
        self._errors: Dict[int, str] = {}   # request id -> why it was aborted

    # ---- admission ------------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        if self.generation_cfg is not None:
            params = self.generation_cfg.fill(params)
        params.validate()
        prompt = [int(t) for t in prompt]
        V = self.runner.plan.vocab_size
        if any(t < 0 or t >= V for t in prompt):
            raise ValueError(f"prompt token ids must lie in [0, {V})")
        max_tokens = params.max_tokens or self.econfig.max_tokens or 16384
        seq_id = self._next_id
        self._next_id += 1
        self.scheduler.add(seq_id, prompt, max_tokens, params.ignore_eos, params.stop_token_ids)
        seed = params.seed if params.seed is not None else (self.seed * 0x9E3779B97F4A7C15 + seq_id + 1)
        self._live[seq_id] = _Live(params, int(seed) & 0xFFFFFFFFFFFFFFFF, len(prompt), time.time())
        return seq_id

    # ---- one iteration --------------------------------------------------------------------------------
    def step(self) -> List[int]:
        """Run one batch to its end; returns the ids of requests that ended with it.

        While a batch of single decode tokens runs on the device, the next one is decided and
        queued behind it (its token ids are read on the device from the running batch's sampled
        tokens), so the device does not wait for the host between decode steps.  A request that
        the running batch ends on a stop token has then one token computed in vain; its result
        is dropped."""
        flight, self._flight = self._flight, None
        ended: List[int] = []
        try:
            if flight is None:
                entries = self.scheduler.schedule()
                ended = self.scheduler.drain_finished()  # requests the scheduler had to abort
                if entries:
                    flight = self._launch(entries, None)
            if flight is not None:
                if self.run_ahead and flight.sampler is not None and not flight.penalties:
                    ahead = self.scheduler.schedule_ahead()
                    if ahead:
                        self._flight = self._launch(ahead, flight)
                        self.stats["steps_decided_ahead"] += 1
                ended += self._retire(flight)
                self.stats["steps"] += 1
        except RuntimeError as e:     # StepError, SchedulerError, KernelError, a CUDA error raised by torch
            ended += self._fail_scheduled(e)
        self.stats["preemptions"] = self.scheduler.preemptions
        for seq_id in ended:
            self._finish(seq_id)
        self._drop_idle_flight()
        return ended

    def _drop_idle_flight(self) -> None:
        """A batch queued for requests that have all ended meanwhile: wait for it, keep nothing."""
        if self._flight is not None and not any(e.req_id in self._live for e in self._flight.wanted):
            try:
                self._retire(self._flight)
            except RuntimeError as e:
                for seq_id in self._fail_scheduled(e):
                    self._finish(seq_id)
            self._flight = None

    def _fail_scheduled(self, error: Exception) -> List[int]:
        """A step failed.  The requests of every batch that is scheduled and not recorded (the one
        that failed and one queued behind it) end as aborted with the reason; their pages go back;
        the device is drained and its error word, scratch and samplers are made ready for the next
        step.  Returns the ids that ended.  Requests that were only waiting are untouched."""
        reason = f"{type(error).__name__}: {error}"
        self.stats["failed_steps"] += 1
        self._flight = None
        ended = self.scheduler.fail_steps()
        for seq_id in ended:
            self._errors[seq_id] = reason
        self.runner.recover()
        for s in self.samplers:
            s.reset()
        return ended

    def _launch(self, entries, after: Optional["_Flight"]) -> "_Flight":
        """Queue a batch and its sampling on the device; nothing waits for it here.  ``after``:
        the batch still running whose sampled tokens are this batch's token ids."""
        inputs = []
        wanted = []
        for e in entries:
            if e.start == 0:
                self.runner.prepare_slot(e.slot)
            tokens = e.tokens if after is None else [self.runner.ahead_token(e.src)]
            inputs.append(StepInput(e.slot, tokens, [len(tokens) - 1] if e.want else []))
            if e.want:
                wanted.append(e)
            if e.start < self._live[e.req_id].prompt_len:
                self.stats["prompt_tokens"] += min(len(e.tokens), self._live[e.req_id].prompt_len - e.start)
        logits = self.runner.step(inputs, allow_graph=self.use_graphs)
        flight = _Flight(wanted=wanted)
        if wanted:
            lives = [self._live[e.req_id] for e in wanted]
            hist = None
            flight.penalties = any(l.params.has_penalties for l in lives)
            if flight.penalties:
                hist = [self.scheduler.tail(e.req_id, PENALTY_HISTORY) if l.params.has_penalties else ()
                        for e, l in zip(wanted, lives)]
            ahead = 1 if after is not None else 0    # tokens of `after` are drawn but not recorded yet
            self._sampler_i ^= 1
            sampler = self.samplers[self._sampler_i]   # two sets of buffers: two batches can be in flight
            flight.tokens_dev = sampler.sample(logits, [l.params for l in lives], [l.seed for l in lives],
                                               [self.scheduler.num_drawn(e.req_id) + ahead for e in wanted], hist)
            sampler.start_copy(flight.tokens_dev)
            flight.sampler = sampler
        return flight

    def _retire(self, flight: "_Flight") -> List[int]:
        """Wait for a queued batch's tokens and record them; returns the ids that ended."""
        sampled: List[int] = []
        if flight.sampler is not None:
            ids, word = flight.sampler.finish_copy()
            sampled = ids.tolist()
            self.runner.raise_on(word)
            now = time.time()
            for e in flight.wanted:
                live = self._live.get(e.req_id)
                if live is not None and not live.t_first:
                    live.t_first = now
            self.stats["decoded_tokens"] += sum(1 for e in flight.wanted if e.req_id in self._live)
        return self.scheduler.commit(sampled)

    def _finish(self, seq_id: int) -> None:
        live = self._live.pop(seq_id, None)
        if live is None:
            return
        out = self.scheduler.output(seq_id)
        now = time.time()
        self._done[seq_id] = GenerationOutput(
            seq_id=seq_id, prompt_length=live.prompt_len, prompt_start_time=_ms(live.t_start),
            decode_start_time=_ms(live.t_first or now), decode_finish_time=_ms(now),
            decoded_length=len(out), decode_output=out, finish_reason=self.scheduler.finish_reason(seq_id),
            error=self._errors.pop(seq_id, None))
        self.scheduler.release(seq_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._flight is not None

    # ---- the reference's calls ----------------------------------------------------------------------------
    def generate_sync(self, params: Union[SamplingParams, Sequence[SamplingParams]],
                      prompts: Sequence[Sequence[int]]) -> List[GenerationOutput]:
        """Generate for every prompt (continuous batching) and return the outputs in prompt order."""
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError(f"{len(params)} sampling params for {len(prompts)} prompts")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while any(i in self._live for i in ids):
            before = (self.stats["steps"], len(self._live))
            self.step()
            if (self.stats["steps"], len(self._live)) == before and not self.has_work():
                break
        return [self._done.pop(i) for i in ids]

    def generate_stream(self, params: SamplingParams, prompt: Sequence[int]) -> Tuple[int, int, "EngineStream"]:
        """Returns (seq_id, prompt_length, stream); the stream yields ``StreamItem``s and can be cancelled."""
        seq_id = self.add_request(prompt, params)
        return seq_id, len(prompt), EngineStream(self, seq_id, len(prompt))

    def cancel(self, seq_id: int) -> bool:
        """End a live request now: its pages go back, its output so far stays readable (finish reason "abort")."""
        if seq_id not in self._live:
            return False
        self.scheduler.abort(seq_id)
        for ended in self.scheduler.drain_finished():
            self._finish(ended)
        self._drop_idle_flight()
        return True

    def get_available_kv_tokens(self) -> int:
        return self.runner.available_kv_tokens()

    def get_num_cached_tokens(self) -> int:
        """Tokens held by a prefix cache; this engine keeps none."""
        return 0
