"""Random tiny configurations of the architecture - head sizes in steps of 16 up to 256, any number
of heads and groups, widths and vocabularies that are no power of two or no multiple of 8, page
sizes from 4 to 64, with and without a window, tied and untied heads - through the step function,
whole and in random portions (some decode steps from CUDA graphs), against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import sharpen

pytestmark = pytest.mark.gpu


def draw_config(rng):
    while True:
        d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 192, 256]))
        nkv = int(rng.choice([1, 2, 3, 4, 5]))
        nh = nkv * int(rng.choice([1, 2, 3, 4, 6, 7, 8, 16, 20]))
        if nh * d <= 4096:
            break
    window = None if rng.random() < 0.6 else int(rng.integers(3, 90))
    return dict(architectures=["Qwen3ForCausalLM"], vocab_size=int(rng.choice([97, 331, 1000, 2053])),
                hidden_size=int(rng.choice([64, 72, 96, 100, 136, 200, 264, 520])),
                intermediate_size=int(rng.choice([64, 88, 176, 200, 344])), num_hidden_layers=int(rng.choice([1, 2, 3])),
                num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d, rms_norm_eps=float(rng.choice([1e-6, 1e-5])),
                rope_theta=float(rng.choice([1e4, 1e6])), max_position_embeddings=512,
                tie_word_embeddings=bool(rng.random() < 0.5), sliding_window=window)


@pytest.mark.parametrize("seed", range(10))
def test_random_configuration_whole_and_in_random_portions(seed, tmp_path):
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.weights import write_random_model
    rng = np.random.default_rng(100 + seed)
    cfg = draw_config(rng)
    page = int(rng.choice([4, 8, 16, 32, 64]))
    n = int(rng.integers(20, 200))
    seq = rng.integers(0, cfg["vocab_size"], size=n).tolist()
    for dtype, store in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        folder = write_random_model(str(tmp_path / dtype), cfg, seed=seed, dtype=store, override=sharpen)
        c, w = plain.load_folder(folder)
        ref = plain.forward(c, w, seq)
        if dtype == "float32":
            tol = 3e-5 * max(1.0, float(ref.abs().max()))
        else:
            tol = 3.0 * float((plain.forward(c, w, seq, round_to=torch.bfloat16) - ref).abs().max())
        r = ModelRunner(folder, dtype, block_size=page, num_blocks=(2 * n) // page + 8, max_num_seqs=2)
        s = r.open_request()
        whole = r.step([StepInput(s, seq, range(n))]).float().cpu().clone()
        r.check_errors()
        r.close_request(s)
        s = r.open_request()
        got, at = [], 0
        while at < n:
            k = min(int(rng.choice([1, 1, 2, 3, 5, 17, 40, 70])), n - at)
            got.append(r.step([StepInput(s, seq[at:at + k], range(k))], allow_graph=bool(rng.random() < 0.5)).float().cpu().clone())
            at += k
        r.check_errors()
        r.close_request(s)
        what = f"{dtype} {cfg} page {page} tokens {n}"
        assert float((whole - ref).abs().max()) <= tol, what
        assert float((torch.cat(got) - ref).abs().max()) <= tol, what
