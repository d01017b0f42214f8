"""The plain implementation itself (no GPU): its parts against independent restatements of the
reference's formulas, and its own float32-vs-float64 gap."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, prompts_for


def test_philox_known_answers():
    # Random123 known-answer vectors for Philox4x32-10
    z = np.zeros(1, np.uint32)
    got = [int(w[0]) for w in plain._philox4x32_10(z, z, z, z, 0, 0)]
    assert got == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = np.full(1, 0xFFFFFFFF, np.uint32)
    got = [int(w[0]) for w in plain._philox4x32_10(f, f, f, f, 0xFFFFFFFF, 0xFFFFFFFF)]
    assert got == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


def test_rope_matches_the_probe_formula():
    # tests/probes/compare_attention_misc_probe.py:33-49 in the reference: rotate halves
    T, heads, d, theta = 11, 3, 8, 10000.0
    x = torch.randn(T, heads, d, dtype=torch.float64)
    pos = [0, 5, 63, 2, 9, 1, 40, 7, 33, 12, 3]
    got = plain.apply_rope(x, plain.rope_angles(pos, d, theta))
    inv = 1.0 / theta ** (np.arange(0, d, 2) / d)
    for t, p in enumerate(pos):
        for j in range(d // 2):
            a = np.float32(np.float32(p) * np.float32(inv[j]))
            c, s = math.cos(a), math.sin(a)
            x1, x2 = x[t, :, j], x[t, :, j + d // 2]
            assert torch.allclose(got[t, :, j], x1 * c - x2 * s, atol=1e-12)
            assert torch.allclose(got[t, :, j + d // 2], x1 * s + x2 * c, atol=1e-12)


def test_norm_swiglu_and_attention_against_direct_sums():
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.randn(12, dtype=torch.float64)
    got = plain.rms_norm(x, w, 1e-5)
    for t in range(5):
        ms = sum(float(v) ** 2 for v in x[t]) / 12
        assert torch.allclose(got[t], x[t] / math.sqrt(ms + 1e-5) * w, atol=1e-12)
    g, u = torch.randn(4, 6, dtype=torch.float64), torch.randn(4, 6, dtype=torch.float64)
    assert torch.allclose(plain.swiglu(g, u), torch.nn.functional.silu(g) * u, atol=1e-12)
    T, nh, nkv, d = 7, 4, 2, 6
    q, k, v = (torch.randn(T, h, d, dtype=torch.float64) for h in (nh, nkv, nkv))
    for window in (None, 3):
        got = plain.causal_attention(q, k, v, 0.5, window)
        for t in range(T):
            for h in range(nh):
                lo = 0 if window is None else max(0, t - window + 1)
                s = [float(q[t, h] @ k[j, h // 2]) * 0.5 for j in range(lo, t + 1)]
                m = max(s)
                p = [math.exp(a - m) for a in s]
                o = sum(pi * v[lo + i, h // 2] for i, pi in enumerate(p)) / sum(p)
                assert torch.allclose(got[t, h], o, atol=1e-12)


def _weights(name, dtype):
    from xinfer_b200.config import Qwen3Config
    from xinfer_b200.models import model_weight_specs
    from xinfer_b200.weights import draw
    from helpers import sharpen_for
    cfg, seed = TINY[name]
    sharpen = sharpen_for(cfg)
    w = {}
    for s in model_weight_specs(Qwen3Config.from_dict(cfg).plan()):
        t = draw(s, seed, 0.02, 0.1, torch.float32)
        t2 = sharpen(s.name, t)
        w[s.name] = (t if t2 is None else t2).to(dtype)
    return cfg, w


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_causality_and_precision_gap(name):
    cfg, w32 = _weights(name, torch.float32)
    _, w64 = _weights(name, torch.float64)
    ids = prompts_for(name, [45])[0]
    full = plain.forward(cfg, w32, ids)
    assert full.shape == (45, cfg["vocab_size"]) and torch.isfinite(full).all()
    # a position's logits depend on no later token
    part = plain.forward(cfg, w32, ids[:20])
    assert torch.allclose(full[:20], part, atol=2e-6)
    ref = plain.forward(cfg, w64, ids)
    gap = (full.double() - ref).abs().max().item()
    assert gap < 2e-5, gap
    # the sharpened weights make attention matter: dropping the window changes windowed logits
    if cfg.get("sliding_window"):
        other = plain.forward(dict(cfg, sliding_window=None), w32, ids)
        assert (other[40:] - full[40:]).abs().max() > 1e-3
        assert torch.allclose(other[: cfg["sliding_window"]], full[: cfg["sliding_window"]], atol=1e-6)
    # bfloat16 rounding at the places an engine stores activations stays near float32
    rb = plain.forward(cfg, w32, ids, round_to=torch.bfloat16)
    assert 1e-4 < (rb - full).abs().max().item() < 0.1


def test_sampling_rules():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=300).astype(np.float32) * 3
    assert plain.sample(logits) == int(np.argmax(logits))
    assert plain.sample(logits, temperature=1e-8, top_k=5) == int(np.argmax(logits))
    tie = logits.copy()
    tie[17] = tie[200] = tie.max() + 1
    assert plain.sample(tie) == 17                                  # lowest index wins a tie
    top5 = set(np.argsort(-logits)[:5].tolist())
    draws = {plain.sample(logits, 1.0, top_k=5, seed=3, draw=n) for n in range(200)}
    assert draws <= top5 and len(draws) > 1
    # nucleus: the kept set is the shortest prefix of the sorted tokens whose mass reaches p
    p = np.exp(logits - logits.max()); p /= p.sum()
    order = np.argsort(-p)
    keep = int(np.searchsorted(np.cumsum(p[order]), 0.6)) + 1
    draws = {plain.sample(logits, 1.0, top_p=0.6, seed=4, draw=n) for n in range(300)}
    assert draws <= set(order[:keep].tolist())
    # the same (seed, draw) gives the same token; the empirical distribution follows softmax
    assert plain.sample(logits, 0.8, seed=9, draw=5) == plain.sample(logits, 0.8, seed=9, draw=5)
    small = np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    counts = np.bincount([plain.sample(small, 1.0, seed=11, draw=n) for n in range(4000)], minlength=4)
    expect = np.exp(small) / np.exp(small).sum()
    assert np.abs(counts / 4000 - expect).max() < 0.03
    pen = plain.apply_penalties(small, [0, 0, 2], frequency=0.5, presence=0.25)
    assert np.allclose(pen, [2.0 - 1.0 - 0.25, 1.0, 0.0 - 0.5 - 0.25, -1.0])


def test_generate_stops_on_eos():
    cfg, w = _weights("A", torch.float32)
    prompt = prompts_for("A", [9])[0]
    out = plain.generate(cfg, w, prompt, 6)
    assert len(out) == 6
    cut = plain.generate(cfg, w, prompt, 6, eos=[out[2]])
    assert cut == out[: out.index(out[2])]
