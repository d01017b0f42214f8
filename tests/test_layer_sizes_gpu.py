"""The real layer sizes of the three published shapes (0.6B, 8B, 32B), with one or two layers and
a small vocabulary, replayed whole, in portions and token by token, and compared with the plain
implementation: the kernels' tilings, split counts and tensor maps at the widths that serving
uses, which the tiny configurations never reach."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TraceBuilder, run_trace, sharpen

pytestmark = pytest.mark.gpu

SHAPES = {
    # name: (hidden, heads, kv heads, head_dim, intermediate, layers, tied, vocab)
    "0.6b": (1024, 16, 8, 128, 3072, 2, True, 1003),
    "8b": (4096, 32, 8, 128, 12288, 1, False, 1201),
    "32b": (5120, 64, 8, 128, 25600, 1, False, 911),
}


@pytest.fixture(scope="module")
def sized_folder(tmp_path_factory):
    from xinfer_b200.weights import write_random_model
    made = {}

    def get(name):
        if name not in made:
            H, nh, nkv, d, inter, layers, tied, vocab = SHAPES[name]
            cfg = dict(architectures=["Qwen3ForCausalLM"], vocab_size=vocab, hidden_size=H, intermediate_size=inter,
                       num_hidden_layers=layers, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d,
                       rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=4096,
                       tie_word_embeddings=tied, sliding_window=None, eos_token_id=1)
            folder = tmp_path_factory.mktemp(f"sized_{name.replace('.', '_')}")
            write_random_model(str(folder), cfg, seed=11, dtype=torch.bfloat16, override=sharpen)
            made[name] = str(folder)
        return made[name]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_real_layer_sizes_match_the_plain_implementation(name, dtype, sized_folder, tmp_path):
    folder = sized_folder(name)
    vocab = SHAPES[name][-1]
    rng = np.random.default_rng(5)
    whole = rng.integers(0, vocab, size=150).tolist()
    cut = rng.integers(0, vocab, size=109).tolist()

    tb = TraceBuilder()
    tb.step([("w", ("whole", 0), 0, whole, True)])
    tb.step([("c", ("cut", 1), 0, cut[:64], True)])
    # a portion beside a single token of the other request, then the last tokens one by one
    tb.step([("c", ("cut", 1), 64, cut[64:101], True), ("w", ("whole", 0), 150, [whole[0]], False)], end=["w"])
    for j in range(101, len(cut)):
        tb.step([("c", ("cut", 1), j, cut[j:j + 1], True)], end=["c"] if j == len(cut) - 1 else [])
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=16)

    cfg, w = plain.load_folder(folder)   # the stored bfloat16 values, widened: both runs see the same weights
    prompts = [whole, cut]
    ref = [plain.forward(cfg, w, p).numpy() for p in prompts]
    if dtype == "float32":
        tol = [2e-5 * max(1.0, float(np.abs(r).max())) for r in ref]
    else:
        tol = [3.0 * np.abs(plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy() - r).max()
               for p, r in zip(prompts, ref)]
    worst = 0.0
    covered = {0: set(), 1: set()}
    for step, rows in tb.rows.items():
        for r, ((mode, i), pos) in enumerate(rows):
            d = float(np.abs(out[step][r] - ref[i][pos]).max())
            worst = max(worst, d)
            assert d <= tol[i], f"{name} {dtype} {mode}: position {pos} (step {step}) differs by {d:.3g} > {tol[i]:.3g}"
            covered[i].add(pos)
    assert covered[0] == set(range(len(whole))) and covered[1] == set(range(len(cut)))
    print(name, dtype, f"worst {worst:.3g} tolerance", [f"{t:.3g}" for t in tol])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_at_real_layer_sizes(dtype, sized_folder, tmp_path):
    """900 tokens at the 0.6B layer sizes, whole and in portions that end inside a 128-query tile and
    inside a 64-key tile: eight query tiles, key/value rings that wrap, cached prefixes of odd lengths."""
    folder = sized_folder("0.6b")
    vocab = SHAPES["0.6b"][-1]
    rng = np.random.default_rng(8)
    whole = rng.integers(0, vocab, size=900).tolist()
    cut = rng.integers(0, vocab, size=900).tolist()
    want_whole = [0, 1, 127, 128, 129, 500, 898, 899]
    tb = TraceBuilder()
    tb.step([("w", ("whole", 0), 0, whole, want_whole)])
    at = 0
    for n in (300, 77, 523):
        last = at + n == len(cut)
        tb.step([("c", ("cut", 1), at, cut[at:at + n], [0, n // 2, n - 1])], end=["c"] if last else [])
        at += n
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=16)
    cfg, w = plain.load_folder(folder)
    prompts = [whole, cut]
    ref = [plain.forward(cfg, w, p).numpy() for p in prompts]
    if dtype == "float32":
        tol = [2e-5 * max(1.0, float(np.abs(r).max())) for r in ref]
    else:
        tol = [3.0 * np.abs(plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy() - r).max() for p, r in zip(prompts, ref)]
    checked = 0
    for step, rows in tb.rows.items():
        for r, ((mode, i), pos) in enumerate(rows):
            d = float(np.abs(out[step][r] - ref[i][pos]).max())
            assert d <= tol[i], f"{dtype} {mode}: position {pos} (step {step}) differs by {d:.3g} > {tol[i]:.3g}"
            checked += 1
    assert checked == len(want_whole) + 9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_depth_at_the_smallest_published_shape(dtype, tmp_path):
    """All 28 layers of the 0.6B shape (a small vocabulary keeps the plain implementation quick):
    200 tokens whole, then 60 token by token.  What only depth shows - error growth over the
    layers in bfloat16, a scratch buffer reused one layer too early - shows here."""
    from xinfer_b200.weights import write_random_model
    H, nh, nkv, d, inter, _, tied, _ = SHAPES["0.6b"]
    vocab, layers = 2003, 28
    cfg = dict(architectures=["Qwen3ForCausalLM"], vocab_size=vocab, hidden_size=H, intermediate_size=inter,
               num_hidden_layers=layers, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d,
               rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=4096,
               tie_word_embeddings=tied, sliding_window=None, eos_token_id=1)
    folder = write_random_model(str(tmp_path / "deep"), cfg, seed=13, dtype=torch.bfloat16, override=sharpen)
    rng = np.random.default_rng(6)
    seq = rng.integers(0, vocab, size=260).tolist()
    tb = TraceBuilder()
    tb.step([("d", ("deep", 0), 0, seq[:200], True)])
    for j in range(200, 260):
        tb.step([("d", ("deep", 0), j, seq[j:j + 1], True)], end=["d"] if j == 259 else [])
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=16)
    cfg_p, w = plain.load_folder(folder)
    ref = plain.forward(cfg_p, w, seq).numpy()
    if dtype == "float32":
        _, w64 = plain.load_folder(folder, dtype=torch.float64)
        own = float(np.abs(plain.forward(cfg_p, w64, seq).float().numpy() - ref).max())
        tol = max(2e-5, 4.0 * own)
    else:
        tol = 3.0 * float(np.abs(plain.forward(cfg_p, w, seq, round_to=torch.bfloat16).numpy() - ref).max())
    worst = 0.0
    for step, rows in tb.rows.items():
        for r, (_, pos) in enumerate(rows):
            dlt = float(np.abs(out[step][r] - ref[pos]).max())
            worst = max(worst, dlt)
            assert dlt <= tol, f"{dtype}: position {pos} (step {step}) differs by {dlt:.3g} > {tol:.3g}"
    assert np.isfinite(ref).all()
    print(f"full depth {dtype}: worst difference {worst:.3g}, tolerance {tol:.3g}")
