"""Device-side sampling for a batch of logits rows: one launch for penalties, one for the draw
(greedy, temperature, top-k, top-p, top-k then top-p; src/utils/logits_processor.rs:258-344)."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels, tracing
from .params import SamplingParams

# tokens that the penalties count: the most recent ones of the request, as many as the reference
# tracks (src/core/runner.rs:1887-1912)
PENALTY_HISTORY = 128


class Sampler:
    def __init__(self, device, max_rows: int, out_dev: Optional[torch.Tensor] = None,
                 err_word: Optional[torch.Tensor] = None):
        """``out_dev``: int32 device buffer of max_rows + 1 that receives the ids (default: one of
        its own).  ``err_word``: a device int32 whose value is copied behind the ids, so that the
        step's tokens and its error word reach the host in one copy (``finish_copy`` returns both)."""
        self.device = device
        self.max_rows = max_rows
        self.err_word = err_word
        rec = kernels.SAMPLE_PARAMS.itemsize
        self._params_host = torch.zeros(max_rows * rec, dtype=torch.uint8, pin_memory=True)
        self._params_dev = torch.zeros(max_rows * rec, dtype=torch.uint8, device=device)
        self._hist_host = torch.zeros(max_rows * PENALTY_HISTORY, dtype=torch.int32, pin_memory=True)
        self._hist_dev = torch.zeros(max_rows * PENALTY_HISTORY, dtype=torch.int32, device=device)
        self._out_dev = out_dev if out_dev is not None else torch.zeros(max_rows + 1, dtype=torch.int32, device=device)
        if self._out_dev.numel() < max_rows + 1 or self._out_dev.dtype != torch.int32:
            raise ValueError("the sampler's output buffer must hold max_rows + 1 int32")
        self._out_host = torch.zeros(max_rows + 1, dtype=torch.int32, pin_memory=True)
        self._scratch = torch.zeros(kernels.sample_scratch_bytes(max_rows), dtype=torch.uint8, device=device)
        self._params_np = self._params_host.numpy().view(kernels.SAMPLE_PARAMS)
        self._hist_np = self._hist_host.numpy()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draws: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """One token per logits row, as an int32 device tensor (a view of a reused buffer).
        ``seeds[r]`` / ``draws[r]``: the request's seed and how many tokens it has drawn before.
        ``histories[r]``: the request's recent tokens, used when it has penalties."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows exceed the sampler's capacity {self.max_rows}")
        rec = self._params_np
        any_pen = False
        off = 0
        for r, p in enumerate(params):
            rec[r]["temperature"] = 0.0 if p.greedy else float(p.temperature)
            rec[r]["top_k"] = int(p.top_k) if p.top_k and p.top_k > 0 else 0
            rec[r]["top_p"] = float(p.top_p) if p.top_p is not None else 1.0
            s = int(seeds[r]) & 0xFFFFFFFFFFFFFFFF
            rec[r]["seed_lo"], rec[r]["seed_hi"] = s & 0xFFFFFFFF, s >> 32
            rec[r]["draw"] = int(draws[r]) & 0xFFFFFFFF
            rec[r]["frequency_penalty"] = float(p.frequency_penalty or 0.0)
            rec[r]["presence_penalty"] = float(p.presence_penalty or 0.0)
            rec[r]["history_offset"] = off
            n = 0
            if p.has_penalties and histories is not None:
                h = list(histories[r])[-PENALTY_HISTORY:]
                n = len(h)
                self._hist_np[off:off + n] = h
                any_pen = any_pen or n > 0
            rec[r]["history_len"] = n
            off += n
        nb = R * kernels.SAMPLE_PARAMS.itemsize
        self._params_dev[:nb].copy_(self._params_host[:nb], non_blocking=True)
        if any_pen:
            self._hist_dev[:off].copy_(self._hist_host[:off], non_blocking=True)
        if tracing.ENABLED:
            tracing.push("sample")
        kernels.sample(self._out_dev, logits, self._params_dev, self._hist_dev, any_pen, self._scratch, self.err_word,
                       capacity=self.max_rows)
        if tracing.ENABLED:
            tracing.pop()
        return self._out_dev[:R]

    def reset(self) -> None:
        """After a failed step: the scratch is zeroed again (a kernel that did not finish may have
        left counters behind) and a queued copy is forgotten."""
        self._scratch.zero_()
        self._copied = 0
        self._copy_done = None

    def to_host(self, tokens_dev: torch.Tensor) -> np.ndarray:
        """Copy sampled ids to the host (synchronises the stream)."""
        self.start_copy(tokens_dev)
        return self.finish_copy()[0]

    def start_copy(self, tokens_dev: torch.Tensor) -> None:
        """Queue the copy of the sampled ids (and the error word behind them) to the host;
        ``finish_copy`` waits for it alone, so work queued after it keeps running."""
        n = tokens_dev.shape[0]
        self._out_host[:n + 1].copy_(self._out_dev[:n + 1], non_blocking=True)
        self._copied = n
        self._copy_done = torch.cuda.Event()
        self._copy_done.record()

    def finish_copy(self):
        """(ids, error word); the word is 0 when the sampler was given none."""
        self._copy_done.synchronize()
        n = self._copied
        return self._out_host[:n].numpy().copy(), (int(self._out_host[n]) if self.err_word is not None else 0)
