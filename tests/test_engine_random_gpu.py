"""Random workloads through the Python entry point in float32 - requests that arrive while others
run, pools barely larger than the longest request (so requests are preempted and recomputed), one to
four request slots, small token budgets and portions, the next step decided ahead or not, greedy,
temperature and top-k sampling, stop tokens - must give exactly the plain implementation's tokens,
and leave the pool whole."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("trial", range(9))
def test_random_workload_equals_plain(trial, model_folders):
    from xinfer_b200 import Engine, EngineConfig, SamplingParams
    rng = np.random.default_rng(7000 + trial)
    name = ["A", "B", "C"][trial % 3]
    cfg, _ = TINY[name]
    folder = model_folders(name, torch.float32)
    c, w = plain.load_folder(folder)
    n_req = int(rng.integers(3, 9))
    prompts = [rng.integers(0, cfg["vocab_size"], size=int(rng.integers(1, 60))).tolist() for _ in range(n_req)]
    params = [SamplingParams(temperature=float(rng.choice([0.0, 0.8])), max_tokens=int(rng.integers(1, 30)),
                             ignore_eos=bool(rng.random() < 0.5), top_k=int(rng.choice([0, 0, 10])), seed=int(rng.integers(0, 1000)))
              for _ in range(n_req)]
    page = PAGE_SIZE[name]
    need = (max(len(p) + sp.max_tokens for p, sp in zip(prompts, params)) + page - 1) // page
    pages = int(rng.integers(need + 1, 2 * need + 2))
    eng = Engine(EngineConfig(weight_path=folder, block_size=page, num_blocks=pages, max_num_seqs=int(rng.integers(1, 5)),
                              max_num_batched_tokens=int(rng.choice([8, 32, 256])), prefill_chunk_size=int(rng.choice([4, 16, 256])),
                              disable_cuda_graph=True, disable_run_ahead=bool(rng.random() < 0.5)), "f32")
    pending, ids = list(range(n_req)), {}
    while pending or eng.has_work():
        while pending and (rng.random() < 0.5 or not eng.has_work()):
            i = pending.pop(0)
            ids[eng.add_request(prompts[i], params[i])] = i
        eng.step()
    eos = cfg.get("eos_token_id")
    eos = [eos] if isinstance(eos, int) else (eos or [])
    for sid, i in ids.items():
        out, sp = eng._done.pop(sid), params[i]
        want = plain.generate(c, w, prompts[i], sp.max_tokens, temperature=sp.temperature, seed=sp.seed, top_k=sp.top_k,
                              eos=[] if sp.ignore_eos else eos)
        assert out.error is None and out.decode_output == want, (name, i, out.finish_reason)
    eng.runner.cache.check_consistent()
    assert eng.runner.cache.free_pages() == pages and eng.runner.cache.live_requests() == 0
