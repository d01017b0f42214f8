"""Tiny configurations and helpers shared by the tests."""
import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three tiny configurations that differ in every size and option: head counts and groups, sizes
# that are no power of two, number of layers, vocabulary, the norms' eps, rope theta, tied or
# untied head, and the window.
TINY: Dict[str, tuple] = {
    "A": (dict(architectures=["Qwen3ForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=128,
               num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
               rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512,
               tie_word_embeddings=True, sliding_window=None, eos_token_id=255), 0),
    "B": (dict(architectures=["Qwen3ForCausalLM"], vocab_size=384, hidden_size=96, intermediate_size=224,
               num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
               rms_norm_eps=1e-5, rope_theta=1000000.0, max_position_embeddings=768,
               tie_word_embeddings=False, sliding_window=None, eos_token_id=[3, 5]), 1),
    "C": (dict(architectures=["Qwen3ForCausalLM"], vocab_size=331, hidden_size=80, intermediate_size=176,
               num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=5, head_dim=48,
               rms_norm_eps=3e-6, rope_theta=50000.0, max_position_embeddings=640,
               tie_word_embeddings=False, sliding_window=37), 2),
}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16}


def sharpen(name: str, t: torch.Tensor):
    """Random N(0, 0.02) weights give nearly flat attention, which would hide a missing key, a
    wrong window edge or a stale page behind the tolerance.  Larger q/k norm weights make the
    scores spread over a few units (their scale is set by the q/k norm weights alone, since the
    norm removes the projections' scale), so every key matters while bfloat16 stays comparable."""
    if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
        return t.float() * 1.7
    return None


def sharpen_for(cfg: dict):
    """``sharpen`` for a configuration.  Where the output head is the embedding table, the most likely
    next token of a random model is the token it was given (a row's product with itself stands far above
    its products with other rows), and greedy generation repeats one token whatever the cache holds; a
    smaller table lets the layers' outputs decide, so that a generated sequence shows a wrong step."""
    if not cfg.get("tie_word_embeddings"):
        return sharpen

    def override(name: str, t: torch.Tensor):
        if name.endswith("embed_tokens.weight"):
            return t.float() * 0.125
        return sharpen(name, t)

    return override


def prompts_for(name: str, lengths: Sequence[int], seed: int = 0) -> List[List[int]]:
    cfg, _ = TINY[name]
    rng = np.random.default_rng(1000 + seed)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]


def run_trace(model_dir: str, dtype: str, steps: List[dict], out_dir: str, max_tokens: int,
              page_size: int = 16, max_num_seqs: int = 8, timeout: int = 600) -> Dict[int, np.ndarray]:
    """Run bin/trace_run on the steps and return {step: logits [wanted, vocab]}."""
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size),
           "--max-num-seqs", str(max_num_seqs)]
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], "every step must be acknowledged in order"
    out = {}
    for s in steps:
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, f"step {s['step']}: {data.size} floats for {wanted} rows of {vocab}"
            out[s["step"]] = data.reshape(wanted, vocab)
        else:
            assert not os.path.exists(path), f"step {s['step']} wanted nothing but wrote a file"
    return out


# ---------------------------------------------------------------------------------------------
# traces for the replay tests
# ---------------------------------------------------------------------------------------------
class TraceBuilder:
    """Collects steps and remembers which (request, position) every wanted row belongs to, and how
    many tokens live requests hold (each rounded up to 64) at the worst moment."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[tuple]] = {}   # step -> [(key, position)]
        self.live: Dict[str, int] = {}
        self.peak = 0

    def step(self, entries, end=()):
        """entries: list of (id, key, start, tokens, want): want is True (every token), False (none) or a
        list of places among these tokens."""
        n = len(self.steps)
        rows, out = [], []
        for rid, key, start, tokens, want in entries:
            w = list(want) if isinstance(want, (list, tuple)) else (list(range(len(tokens))) if want else [])
            out.append({"id": rid, "tokens": list(tokens), "want": w})
            rows += [(key, start + i) for i in w]
            self.live[rid] = self.live.get(rid, 0) + len(tokens)
        self.peak = max(self.peak, sum((v + 63) // 64 * 64 for v in self.live.values()))
        self.steps.append({"step": n, "entries": out, "end": list(end)})
        if rows:
            self.rows[n] = rows
        for rid in end:
            self.live.pop(rid, None)
        return n


def cut_sizes(total: int, pattern: Sequence[int]) -> List[int]:
    out, i = [], 0
    while total > 0:
        n = min(pattern[i % len(pattern)], total)
        if total - n == 1:      # never leave a single token for a "portion"
            n += 1
        out.append(n)
        total -= n
        i += 1
    return out


def build_all_modes(prompts: List[List[int]], seed: int = 0):
    """One trace with the four ways of cutting, for prompts[i] as request i:
    whole / most in one step then the last 32 one by one / portions of changing size down to two
    tokens / mixed, up to four live requests with portions beside single tokens."""
    import random
    rng = random.Random(seed)
    tb = TraceBuilder()
    for i, p in enumerate(prompts):                       # 1. whole
        tb.step([(f"w{i}", ("whole", i), 0, p, True)], end=[f"w{i}"])
    for i, p in enumerate(prompts):                       # 2. the last 32 one by one
        head = max(len(p) - 32, 1)
        tb.step([(f"t{i}", ("tail", i), 0, p[:head], True)])
        for j in range(head, len(p)):
            tb.step([(f"t{i}", ("tail", i), j, p[j:j + 1], True)], end=[f"t{i}"] if j == len(p) - 1 else [])
        if head == len(p):
            tb.steps[-1]["end"] = [f"t{i}"]
            tb.live.pop(f"t{i}", None)
    for i, p in enumerate(prompts):                       # 3. portions of changing size
        pat = [[2, 7, 3, 16, 2, 29, 5, 11], [13, 2, 2, 40, 3, 9], [5, 2, 31, 2, 17]][i % 3]
        at = 0
        for n in cut_sizes(len(p), pat):
            last = at + n == len(p)
            tb.step([(f"c{i}", ("portions", i), at, p[at:at + n], True)], end=[f"c{i}"] if last else [])
            at += n
    # 4. mixed: requests arrive while others run; each brings prompt portions, then its last 12
    #    tokens one by one beside the portions of others; a request may sit a step out
    order = list(range(len(prompts))) + list(range(len(prompts)))   # every request twice, so pages cycle
    waiting = [(f"m{k}", i) for k, i in enumerate(order)]
    live = {}
    while waiting or live:
        while waiting and len(live) < 4 and (not live or rng.random() < 0.6):
            rid, i = waiting.pop(0)
            live[rid] = [i, 0]
        chosen = [rid for rid in live if rng.random() < 0.8] or [next(iter(live))]
        entries, ended = [], []
        for rid in chosen:
            i, at = live[rid]
            p = prompts[i]
            left = len(p) - at
            n = 1 if left <= 12 else min(rng.choice([2, 3, 5, 9, 17, 33]), left - 12)
            entries.append((rid, ("mixed", i), at, p[at:at + n], True))
            live[rid][1] = at + n
            if at + n == len(p):
                ended.append(rid)
        tb.step(entries, end=ended)
        for rid in ended:
            del live[rid]
    return tb


def replay_in_process(runner, steps: List[dict]) -> Dict[int, np.ndarray]:
    """What bin/trace_run does, inside this process: for models whose parts a test has registered
    (a child process would not know them).  Returns {step: logits [wanted, vocab]}."""
    from xinfer_b200.engine.runner import StepInput
    slots, out = {}, {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = runner.open_request()
            entries.append(StepInput(slots[e["id"]], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            runner.check_errors()
            if logits.shape[0]:
                out[s["step"]] = logits.float().cpu().numpy().copy()
        for rid in s.get("end", []):
            if rid in slots:
                runner.close_request(slots.pop(rid))
    assert not slots, "every request of a trace must end"
    return out
