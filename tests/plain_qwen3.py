"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache, one function
per part, on the CPU.  It shares no code with the engine (it reads safetensors through the
``safetensors`` package, not the engine's reader) and is the oracle of the tests.

It rests on the formulas of the reference's sources (cited per function as file:line inside the
reference project): the reference's own model code cannot be imported or compiled here (a Rust
crate whose tensor and kernel layers are external git crates; no Rust toolchain, no network), so
no output of the reference's model exists under tests/golden.  What can be run of the reference
on the CPU are the Python golden functions of its differential probes - rotation, SiLU gate,
causal attention with grouped heads after a prefix; their outputs on small seeded inputs are in
tests/golden/probe_parts.safetensors (written by tests/golden/make_golden.py), and
tests/test_golden.py holds ``apply_rope``, ``swiglu`` and ``causal_attention`` against them.  RMSNorm, the
order of q/k norm and rotation, the residual structure and the output head are pinned by reading alone.

``dtype`` float64 gives a high-precision run whose rotation angles are still the float32 values
the reference computes; float32 is the like-for-like run.  ``round_to`` = torch.bfloat16 rounds
weights-free activations at the places where a bfloat16 engine stores them, to measure how far a
faithful bfloat16 run may drift from float32.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------
# loading
# ---------------------------------------------------------------------------------------------
def load_folder(model_dir: str, dtype=torch.float32):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


def _round(x: torch.Tensor, round_to) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


# ---------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------
def embed(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """x0[t] = E[id[t]], no scaling.  src/models/qwen3.rs:302-309, 332-336."""
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, plain weight (not 1 + w).
    src/models/layers/others.rs:22-46, 65-85; is_gemma=false at src/models/qwen3.rs:84."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x . W^T, W stored [out, in], no bias.  src/models/layers/linear.rs:76-124."""
    return x @ w.t()


def rope_angles(positions: Sequence[int], head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq_j = 1 / theta^(2j/d) from a float64 power rounded to float32; angle = pos *
    inv_freq in float32.  src/models/layers/rotary_emb.rs:42-58."""
    j = np.arange(0, head_dim, 2, dtype=np.float64)
    inv = (np.float32(1.0) / np.power(np.float64(theta), j / np.float64(head_dim)).astype(np.float32)).astype(np.float32)
    pos = np.asarray(list(positions), dtype=np.float32)
    return torch.from_numpy((pos[:, None] * inv[None, :]).astype(np.float32))  # [T, d/2]


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """NeoX halves: (x_j, x_{j+d/2}) <- (x_j cos - x_{j+d/2} sin, x_j sin + x_{j+d/2} cos).
    x: [T, heads, d].  src/models/layers/rotary_emb.rs:76-105 with is_rope_i=false
    (src/utils/mod.rs:2303); formula as in tests/probes/compare_attention_misc_probe.py:33-49."""
    half = x.shape[-1] // 2
    # cos/sin of the float32 angle, evaluated in float64 and used in x's precision
    cos = torch.cos(angles.double()).to(x.dtype)[:, None, :]
    sin = torch.sin(angles.double()).to(x.dtype)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, d], k/v [T, nkv, d]; query head h uses kv head h // (nh / nkv)
    (src/models/layers/attention.rs:1040-1047); s = (q . k) * scale, causal, softmax, P v
    (dense form as in tests/probes/compare_flashinfer_probe.py:51-73; scale 1/sqrt(d) at
    src/models/layers/attention.rs:691).  With a window, position p sees keys j with
    p - window < j <= p (the reference passes ``sliding_window`` to its external attention
    kernels, src/models/layers/attention.rs:693; the bound is the usual one for that option)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    idx = torch.arange(T)
    allowed = idx[None, :] <= idx[:, None]
    if window is not None:
        allowed &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kh = k[:, h // g, :]
        vh = v[:, h // g, :]
        s = (q[:, h, :] @ kh.t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(z) = z / (1 + exp(-z)).  src/models/layers/mlp.rs:620-631;
    tests/probes/compare_attention_misc_probe.py:81-83."""
    return gate / (1.0 + torch.exp(-gate)) * up


# ---------------------------------------------------------------------------------------------
# the decoder
# ---------------------------------------------------------------------------------------------
def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: dict,
                    positions: Sequence[int], round_to=None) -> torch.Tensor:
    """q/k/v projections, per-head RMSNorm of q and k before the rotation, rotation, attention,
    output projection.  src/models/layers/attention.rs:796-977 (norm :709-748, :869)."""
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg["rms_norm_eps"]
    T = h.shape[0]
    q = _round(linear(h, w[p + "q_proj.weight"]), round_to).view(T, nh, d)
    k = _round(linear(h, w[p + "k_proj.weight"]), round_to).view(T, nkv, d)
    v = _round(linear(h, w[p + "v_proj.weight"]), round_to).view(T, nkv, d)
    q = rms_norm(q, w[p + "q_norm.weight"], eps)
    k = rms_norm(k, w[p + "k_norm.weight"], eps)
    ang = rope_angles(positions, d, cfg.get("rope_theta") or 10000.0)
    q = _round(apply_rope(q, ang), round_to)
    k = _round(apply_rope(k, ang), round_to)
    o = _round(causal_attention(q, k, v, 1.0 / math.sqrt(d), cfg.get("sliding_window")), round_to)
    return _round(linear(o.reshape(T, nh * d), w[p + "o_proj.weight"]), round_to)


def mlp_block(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, round_to=None) -> torch.Tensor:
    """down( silu(gate(h)) * up(h) ).  src/models/layers/mlp.rs:613-697."""
    g = _round(linear(h, w[p + "gate_proj.weight"]), round_to)
    u = _round(linear(h, w[p + "up_proj.weight"]), round_to)
    return _round(linear(_round(swiglu(g, u), round_to), w[p + "down_proj.weight"]), round_to)


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict,
                  positions: Sequence[int], round_to=None) -> torch.Tensor:
    """x + attn(norm(x)), then + mlp(norm(.)).  src/models/qwen3.rs:108-134."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    h = _round(rms_norm(x, w[p + "input_layernorm.weight"], eps), round_to)
    a = attention_block(h, w, p + "self_attn.", cfg, positions, round_to)
    r1 = _round(x + a, round_to)
    h2 = _round(rms_norm(r1, w[p + "post_attention_layernorm.weight"], eps), round_to)
    f = mlp_block(h2, w, p + "mlp.", round_to)
    return _round(r1 + f, round_to)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], round_to=None) -> torch.Tensor:
    """Logits [T, vocab] for a whole sequence at positions 0..T-1.
    src/models/qwen3.rs:311-374: embedding, the layers, final norm, head (tied: the embedding
    table, :267-287)."""
    x = embed(ids, w["model.embed_tokens.weight"])
    positions = list(range(len(ids)))
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions, round_to)
    y = _round(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), round_to)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return linear(y, head)


# ---------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------
def _philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Philox4x32 with 10 rounds on numpy uint32 arrays (counter words c0..c3, key k0, k1)."""
    M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32).copy() for c in (c0, c1, c2, c3))
    k0, k1 = np.uint32(k0), np.uint32(k1)
    for _ in range(10):
        p0 = M0 * c0.astype(np.uint64)
        p1 = M1 * c2.astype(np.uint64)
        hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), p0.astype(np.uint32)
        hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), p1.astype(np.uint32)
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = np.uint32((int(k0) + 0x9E3779B9) & 0xFFFFFFFF)
        k1 = np.uint32((int(k1) + 0xBB67AE85) & 0xFFFFFFFF)
    return c0, c1, c2, c3


def gumbel_noise(seed: int, draw: int, vocab: int) -> np.ndarray:
    """G_i = -log(-log(u_i)), u_i from Philox keyed by the request's seed with counter
    (i // 4, draw, tag, 0), word i % 4, mapped to (0, 1) through its top 23 bits."""
    n4 = (vocab + 3) // 4
    idx = np.arange(n4, dtype=np.uint32)
    words = _philox4x32_10(idx, np.full(n4, draw, np.uint32), np.full(n4, 0x58494E46, np.uint32),
                           np.zeros(n4, np.uint32), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    w = np.stack(words, axis=1).reshape(-1)[:vocab]
    u = ((w >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
    return (-np.log(-np.log(u))).astype(np.float32)


def apply_penalties(logits: np.ndarray, history: Sequence[int], frequency: float, presence: float) -> np.ndarray:
    """logit -= count * frequency + (count > 0) * presence over the history tokens.
    src/utils/logits_processor.rs:358-378."""
    out = logits.astype(np.float32).copy()
    counts: Dict[int, int] = {}
    for t in history:
        if 0 <= t < len(out):
            counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        out[t] = np.float32(out[t] - np.float32(c) * np.float32(frequency) - np.float32(presence))
    return out


def sample(logits: np.ndarray, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
           seed: int = 0, draw: int = 0) -> int:
    """The reference's strategies (src/utils/logits_processor.rs:48-65): temperature < 1e-7 is
    argmax; else softmax(logits / T) over all tokens, over the k largest (top-k), over the
    nucleus (top-p: walking down the sorted candidates, a candidate is kept while the mass before
    it is < p, :92-101), or top-k then top-p on the renormalised k (:173-195).  Top-p alone looks
    at the 256 largest, as the reference's device sampler does (:268-275).  The draw itself is
    argmax(logit / T + Gumbel noise) over the kept tokens, which has the softmax distribution."""
    logits = np.asarray(logits, dtype=np.float32)
    V = logits.shape[0]
    if not (temperature >= 1e-7):
        return int(np.argmax(logits))
    inv_t = np.float32(1.0) / np.float32(temperature)
    noise = gumbel_noise(seed, draw, V)
    use_p = 0.0 < top_p < 1.0
    if top_k <= 0 and not use_p:
        return int(np.argmax(logits * inv_t + noise))
    k = min(top_k if top_k > 0 else 256, 1024, V)
    order = sorted(range(V), key=lambda i: (-logits[i], i))[:k]  # value down, then lower index
    cand = np.asarray(order)
    keep = len(cand)
    if use_p:
        p = np.exp((logits[cand] - logits[cand[0]]) * inv_t).astype(np.float32)
        total = np.float32(0)
        for x in p:
            total = np.float32(total + x)
        cum, keep = np.float32(0), 0
        for x in p:
            if cum >= np.float32(top_p):
                break
            cum = np.float32(cum + np.float32(x / total))
            keep += 1
    cand = cand[:keep]
    vals = logits[cand] * inv_t + noise[cand]
    best = np.flatnonzero(vals == vals.max())
    return int(cand[best].min())


def generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], steps: int, *,
             temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
             eos: Sequence[int] = (), round_to=None) -> List[int]:
    """Whole-sequence recomputation for every new token; returns the generated ids (a token in
    ``eos`` ends generation and stays out, src/core/scheduler.rs:617-647)."""
    ids = list(prompt)
    out: List[int] = []
    for n in range(steps):
        logits = forward(cfg, w, ids, round_to)[-1].float().numpy()
        tok = sample(logits, temperature, top_k, top_p, seed, n)
        if tok in eos:
            break
        ids.append(tok)
        out.append(tok)
    return out
