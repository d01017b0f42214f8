"""Trace replay on the GPU: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests over a pool so small that pages are used
again - in float32 and bfloat16, every position compared with the plain implementation."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import PAGE_SIZE, build_all_modes, prompts_for, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 45, 130, 33], "B": [97, 41, 64, 150], "C": [120, 39, 75, 58]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_way_of_cutting_gives_the_plain_logits(name, dtype, model_folders, tmp_path):
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = model_folders(name, store)
    prompts = prompts_for(name, LENGTHS[name])
    tb = build_all_modes(prompts, seed=len(name))
    assert max(len(s["entries"]) for s in tb.steps) >= 3, "the mixed mode must batch several requests"
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=PAGE_SIZE[name])

    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in prompts]
    if dtype == "float32":
        # the plain implementation's own float32 error against float64 is a few 1e-7 here
        tol = [2e-5] * len(prompts)
    else:
        # how far a faithful bfloat16 run drifts: the plain implementation with activations
        # rounded to bfloat16 where an engine stores them
        tol = [3.0 * np.abs(plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy() - r).max()
               for p, r in zip(prompts, ref)]
    seen = {}
    worst = {}
    for step, rows in tb.rows.items():
        got = out[step]
        assert got.shape[0] == len(rows)
        for r, ((mode, i), pos) in enumerate(rows):
            d = float(np.abs(got[r] - ref[i][pos]).max())
            worst[mode] = max(worst.get(mode, 0.0), d)
            assert d <= tol[i], (f"{name} {dtype} {mode}: request {i} position {pos} (step {step}) differs by {d:.3g} "
                                 f"> {tol[i]:.3g}; first wrong token of this mode")
            seen.setdefault((mode, i), {}).setdefault(pos, []).append(got[r])
    # every mode covered every position of every request
    for mode in ("whole", "tail", "portions", "mixed"):
        for i, p in enumerate(prompts):
            assert sorted(seen[(mode, i)]) == list(range(len(p))), (mode, i)
    if dtype == "float32":
        # float32 reductions never depend on how the batch was cut: the modes agree bit for bit
        for (mode, i), by_pos in seen.items():
            for pos, rows in by_pos.items():
                base = seen[("whole", i)][pos][0]
                for r in rows:
                    assert np.array_equal(r, base), f"{mode} request {i} position {pos} is not bit-identical to the whole run"
    print(name, dtype, "worst difference per mode:", {k: f"{v:.3g}" for k, v in worst.items()}, "tolerance", [f"{t:.3g}" for t in tol])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_freed_pages_are_poisoned_and_nothing_reads_them(name, dtype, model_folders):
    """The debug mode that fills every freed page with NaN in every layer before the next step: the
    four ways of cutting over a pool so small that pages cycle (configuration C also gives pages back
    behind its window) must still give the plain logits - no kernel reads a page it does not own."""
    from helpers import replay_in_process
    from xinfer_b200.engine.runner import ModelRunner
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = model_folders(name, store)
    prompts = prompts_for(name, LENGTHS[name])
    tb = build_all_modes(prompts, seed=len(name))
    page = PAGE_SIZE[name]
    runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=8,
                         poison_freed_pages=True)
    out = replay_in_process(runner, tb.steps)
    assert runner.pages_poisoned > runner.num_blocks, "pages must have been freed, poisoned and used again"
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in prompts]
    tol = [2e-5 if dtype == "float32" else 3.0 * np.abs(plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy() - r).max()
           for p, r in zip(prompts, ref)]
    for step, rows in tb.rows.items():
        assert np.isfinite(out[step]).all(), f"step {step} read a poisoned page"
        for r, ((mode, i), pos) in enumerate(rows):
            assert float(np.abs(out[step][r] - ref[i][pos]).max()) <= tol[i], (mode, i, pos)
