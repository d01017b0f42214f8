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


def test_the_same_wave_again_gives_the_same_tokens_and_holds_no_more_memory(model_folders):
    # bfloat16 with CUDA graphs and steps decided ahead: five times the same twelve requests (temperature and
    # greedy, arriving while others run) through one engine.  From the second wave on everything is reused -
    # pages that others have held, captured graphs, workspaces, samplers' buffers - so the tokens must be those
    # of the first wave, and the device memory in use must stay where the first wave left it.
    from xinfer_b200 import Engine, EngineConfig, SamplingParams
    cfg, _ = TINY["B"]
    folder = model_folders("B", torch.bfloat16)
    page = PAGE_SIZE["B"]
    eng = Engine(EngineConfig(weight_path=folder, block_size=page, num_blocks=24, max_num_seqs=4, max_num_batched_tokens=64,
                              prefill_chunk_size=24), "bf16")
    waves, held = [], []
    for wave in range(5):
        rng = np.random.default_rng(99)
        prompts = [rng.integers(0, cfg["vocab_size"], size=int(rng.integers(1, 70))).tolist() for _ in range(12)]
        params = [SamplingParams(temperature=float(rng.choice([0.0, 0.9])), max_tokens=int(rng.integers(2, 40)), ignore_eos=True,
                                 seed=int(rng.integers(0, 1000))) for _ in range(12)]
        pending, ids = list(range(12)), {}
        while pending or eng.has_work():
            while pending and (rng.random() < 0.4 or not eng.has_work()):
                i = pending.pop(0)
                ids[eng.add_request(prompts[i], params[i])] = i
            eng.step()
        outs = {i: eng._done.pop(sid) for sid, i in ids.items()}
        assert all(o.error is None and o.decoded_length == params[i].max_tokens for i, o in outs.items())
        waves.append([outs[i].decode_output for i in range(12)])
        torch.cuda.synchronize()
        held.append(torch.cuda.memory_allocated())
        eng.runner.cache.check_consistent()
        assert eng.runner.cache.free_pages() == 24 and eng.runner.cache.live_requests() == 0
    assert all(w == waves[0] for w in waves[1:])
    assert held[1:] == [held[1]] * 4 and held[1] <= held[0] + (1 << 20), held
    assert eng.stats["preemptions"] > 0 and eng.stats["steps_decided_ahead"] > 0, eng.stats     # the waves met both
