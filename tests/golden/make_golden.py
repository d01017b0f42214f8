#!/usr/bin/env python3
"""Writes tests/golden/probe_parts.safetensors: outputs of the reference project's OWN golden functions -
the independent PyTorch references of its differential probes - on small seeded inputs, beside those inputs.

    python tests/golden/make_golden.py --reference <root of the reference project>

The reference's model code is Rust and cannot be imported or compiled here, but its probe scripts carry
Python references for three parts of the Qwen3 layer, and those can be run on the CPU:

* ``rope`` of tests/probes/compare_attention_misc_probe.py (rotation of q and k by cos / sin tables looked up
  at positions, NeoX halves or interleaved pairs),
* the SiLU gate expression of the same file's ``main`` (``silu(gate) * up`` of a packed gate/up row),
* ``dense_fp32`` of tests/probes/compare_flashinfer_probe.py (causal attention with grouped heads for queries
  appended after a prefix).

The functions are taken from the reference's files when this script runs (their text is parsed and executed
here; nothing of it is stored), so the committed file holds numbers only.  tests/test_golden.py compares
the plain implementation's parts with them; it needs no reference at hand.
"""
import argparse
import ast
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def function_from(path: str, name: str):
    """The top-level function ``name`` of the Python file at ``path``, compiled alone."""
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            module = ast.Module(body=[node], type_ignores=[])
            scope = {"torch": torch, "F": F}
            exec(compile(module, path, "exec"), scope)
            return scope[name]
    raise SystemExit(f"{path} has no function {name}")


def silu_gate_expression(path: str):
    """The expression the misc probe's main() uses for the SiLU gate of bfloat16 rows, as a function of
    (gate_up, n): the first assignment to ``expected`` whose value calls F.silu."""
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    for node in ast.walk(tree):
        if (isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name)
                and node.targets[0].id == "expected" and "F.silu" in ast.unparse(node.value)):
            code = compile(ast.Expression(node.value), path, "eval")
            return lambda gate_up, n: eval(code, {"torch": torch, "F": F, "gate_up": gate_up, "n": n})
    raise SystemExit(f"{path}: the SiLU gate expression was not found")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference project")
    ap.add_argument("--out", default=os.path.join(HERE, "probe_parts.safetensors"))
    args = ap.parse_args()
    probes = os.path.join(args.reference, "tests", "probes")
    rope = function_from(os.path.join(probes, "compare_attention_misc_probe.py"), "rope")
    silu_gate = silu_gate_expression(os.path.join(probes, "compare_attention_misc_probe.py"))
    dense = function_from(os.path.join(probes, "compare_flashinfer_probe.py"), "dense_fp32")

    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(20260101)
    out = {}

    # ---- rotation: 11 tokens at scattered positions, 3 query heads and 1 key head of 16; tables of 40 positions
    d, positions = 16, torch.tensor([0, 1, 2, 7, 7, 13, 21, 22, 30, 38, 39], dtype=torch.int32)
    inv = (np.float32(1.0) / np.power(np.float64(10000.0), np.arange(0, d, 2, dtype=np.float64) / d).astype(np.float32))
    angles = torch.from_numpy((np.arange(40, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32))
    cos, sin = torch.cos(angles.double()).float(), torch.sin(angles.double()).float()
    q, k = torch.randn(11, 3, d, generator=g), torch.randn(11, 1, d, generator=g)
    for tag, interleaved in (("neox", False), ("interleaved", True)):
        q_out, k_out = rope(q, k, cos, sin, positions, interleaved)
        out[f"rope.{tag}.q_out"], out[f"rope.{tag}.k_out"] = q_out.float().contiguous(), k_out.float().contiguous()
    out.update({"rope.q": q, "rope.k": k, "rope.cos": cos, "rope.sin": sin, "rope.positions": positions, "rope.angles": angles})

    # ---- the SiLU gate: 5 rows of 24 gate and 24 up values, bfloat16 in and out as in the probe
    gate_up = (torch.randn(5, 48, generator=g) * 3).to(torch.bfloat16)
    out["silu.gate_up"] = gate_up.float()
    out["silu.out"] = silu_gate(gate_up, 24).float().contiguous()

    # ---- attention: 9 queries appended after a prefix of 5, 6 query heads over 2 key/value heads of 16
    case = {"prefix": 5, "append": 9, "hq": 6, "hkv": 2, "dim": 16, "fp8": False,
            "q": torch.randn(9, 6, 16, generator=g), "k": torch.randn(14, 2, 16, generator=g), "v": torch.randn(14, 2, 16, generator=g)}
    out["attention.out"] = dense(case, torch.device("cpu")).float().contiguous()
    for name in ("q", "k", "v"):
        out[f"attention.{name}"] = case[name].to(torch.bfloat16).float()      # what the probe computes on
    out["attention.prefix"] = torch.tensor([5], dtype=torch.int32)

    save_file({k: v.contiguous() for k, v in out.items()}, args.out)
    print(f"wrote {args.out}: {len(out)} tensors, {os.path.getsize(args.out)} bytes")

    # the comparison the test makes, once here
    sys.path.insert(0, os.path.join(HERE, ".."))
    import test_golden
    test_golden.compare_all(args.out, verbose=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
