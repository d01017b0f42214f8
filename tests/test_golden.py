"""The plain implementation's parts against outputs of the reference project's own Python golden functions
(tests/golden/probe_parts.safetensors, written by tests/golden/make_golden.py): rotation, SiLU gate, causal
attention with grouped heads after a prefix.  No GPU, no reference at hand."""
import os

import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "probe_parts.safetensors")


def compare_all(path: str = GOLDEN, verbose: bool = False):
    from safetensors.torch import load_file
    t = load_file(path)
    worst = {}
    # rotation, NeoX halves (the layout Qwen3 uses): the tables' angles are those of rope_angles
    ang = plain.rope_angles(range(40), 16, 10000.0)
    assert torch.equal(ang, t["rope.angles"])
    at = ang[t["rope.positions"].long()]
    for name in ("q", "k"):
        got = plain.apply_rope(t[f"rope.{name}"], at)
        worst[f"rope.{name}"] = (got - t[f"rope.neox.{name}_out"]).abs().max().item()
        assert worst[f"rope.{name}"] <= 1e-6
        # and the interleaved layout is not what the plain implementation (or Qwen3) applies
        assert (got - t[f"rope.interleaved.{name}_out"]).abs().max().item() > 1e-2
    # the SiLU gate, rounded to bfloat16 as the probe's expression rounds it: one unit in the last place at most
    gu = t["silu.gate_up"]
    got = plain.swiglu(gu[:, :24], gu[:, 24:]).to(torch.bfloat16).float()
    ulp = torch.maximum(t["silu.out"].abs(), torch.tensor(1e-30)) * 2.0 ** -7
    worst["silu"] = ((got - t["silu.out"]).abs() / ulp).max().item()
    assert worst["silu"] <= 1.0
    # attention: the appended queries' rows of a whole-sequence run (the prefix's queries are not asked for)
    prefix = int(t["attention.prefix"][0])
    k, v = t["attention.k"], t["attention.v"]
    q = torch.cat([torch.zeros(prefix, *t["attention.q"].shape[1:]), t["attention.q"]])
    got = plain.causal_attention(q, k, v, 1.0 / 16 ** 0.5)[prefix:]
    worst["attention"] = (got - t["attention.out"]).abs().max().item()
    assert worst["attention"] <= 2e-6
    if verbose:
        print("largest differences from the reference's golden functions:", worst)
    return worst


def test_plain_parts_equal_the_references_golden_functions():
    compare_all()
