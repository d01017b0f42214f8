"""The sampling kernel against the plain sampler: same seeds, same draws, same tokens."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def run(logits, params, seeds, draws, histories=None):
    from xinfer_b200.sampling import Sampler
    dev = torch.device("cuda:0")
    s = Sampler(dev, max_rows=len(params))
    return s.to_host(s.sample(torch.tensor(logits, device=dev), params, seeds, draws, histories)).tolist()


@pytest.mark.parametrize("vocab", [5, 331, 5000, 151936])
def test_greedy_and_temperature(vocab):
    from xinfer_b200.sampling import SamplingParams
    rng = np.random.default_rng(vocab)
    R = 6
    logits = (rng.normal(size=(R, vocab)) * 2).astype(np.float32)
    logits[1, [vocab // 3, vocab - 1]] = logits[1].max() + 1          # a tie: the lower index wins
    params = [SamplingParams(), SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, seed=1),
              SamplingParams(temperature=1.0, seed=2), SamplingParams(temperature=1.5, seed=3), SamplingParams(temperature=1e-9)]
    seeds = [0, 0, 1, 2, 3 + (5 << 32), 0]
    for draw in (0, 1, 77):
        got = run(logits, params, seeds, [draw] * R)
        want = [plain.sample(logits[r], params[r].temperature or 0.0, seed=seeds[r], draw=draw) for r in range(R)]
        assert got == want
    assert run(logits, params, seeds, [0] * R)[1] == vocab // 3


@pytest.mark.parametrize("vocab", [40, 1031, 151936])
def test_top_k_top_p_and_both(vocab):
    from xinfer_b200.sampling import SamplingParams
    rng = np.random.default_rng(vocab + 1)
    combos = [(1, None), (5, None), (50, None), (1024, None), (None, 0.3), (None, 0.9), (20, 0.5), (300, 0.95), (7, 1.0), (0, 0.0)]
    R = len(combos)
    logits = (rng.normal(size=(R, vocab)) * 3).astype(np.float32)
    # coarse values (as a bfloat16 head produces) make ties at the k-th place common
    logits = np.round(logits * 8) / 8
    params = [SamplingParams(temperature=0.9, top_k=k, top_p=p) for k, p in combos]
    seeds = list(range(100, 100 + R))
    for draw in range(12):
        got = run(logits, params, seeds, [draw] * R)
        want = [plain.sample(logits[r], 0.9, top_k=combos[r][0] or 0, top_p=combos[r][1] if combos[r][1] is not None else 1.0,
                             seed=seeds[r], draw=draw) for r in range(R)]
        assert got == want, (draw, got, want)


def test_penalties_and_batch_independence():
    from xinfer_b200.sampling import SamplingParams
    vocab, R = 500, 4
    rng = np.random.default_rng(3)
    logits = (rng.normal(size=(R, vocab))).astype(np.float32)
    hist = [rng.integers(0, 30, size=n).tolist() for n in (0, 5, 128, 200)]
    params = [SamplingParams(temperature=0.8, frequency_penalty=0.7, presence_penalty=0.4, seed=r) for r in range(R)]
    got = run(logits.copy(), params, list(range(R)), [3] * R, hist)
    want = [plain.sample(plain.apply_penalties(logits[r], hist[r][-128:], 0.7, 0.4), 0.8, seed=r, draw=3) for r in range(R)]
    assert got == want
    # a row's token does not depend on the rows beside it
    alone = [run(logits[r:r + 1].copy(), [params[r]], [r], [3], [hist[r]])[0] for r in range(R)]
    assert alone == got


def test_distribution_follows_softmax():
    from xinfer_b200.sampling import SamplingParams
    small = np.array([[2.0, 1.0, 0.0, -1.0, 0.5]], dtype=np.float32)
    n = 3000
    toks = run(np.repeat(small, n, 0), [SamplingParams(temperature=1.0)] * n, [42] * n, list(range(n)))
    freq = np.bincount(toks, minlength=5) / n
    expect = np.exp(small[0]) / np.exp(small[0]).sum()
    assert np.abs(freq - expect).max() < 0.03


@pytest.mark.parametrize("mode", ["topk_topp", "greedy", "top_p_alone"])
def test_one_sampler_over_shrinking_and_growing_batches(mode):
    """One sampler (one scratch buffer, laid out for its capacity) serves batches of changing
    size, as the engine's does while requests end: the counters of a smaller batch must not fall
    where a larger batch left candidates or partial results."""
    from xinfer_b200.sampling import Sampler, SamplingParams
    dev = torch.device("cuda:0")
    vocab = 5003
    s = Sampler(dev, max_rows=17)
    rng = np.random.default_rng(11)
    if mode == "topk_topp":
        p = SamplingParams(temperature=0.9, top_k=32, top_p=0.95)
    elif mode == "top_p_alone":
        p = SamplingParams(temperature=0.9, top_p=0.9)
    else:
        p = SamplingParams()
    for draw, R in enumerate([8, 7, 3, 1, 17, 16, 9, 17, 2]):
        logits = np.round(rng.normal(size=(R, vocab)) * 3 * 8).astype(np.float32) / 8
        seeds = list(range(50, 50 + R))
        got = s.to_host(s.sample(torch.tensor(logits, device=dev), [p] * R, seeds, [draw] * R)).tolist()
        want = [plain.sample(logits[r], p.temperature or 0.0, top_k=p.top_k or 0,
                             top_p=p.top_p if p.top_p is not None else 1.0, seed=seeds[r], draw=draw) for r in range(R)]
        assert got == want, (R, got, want)


@pytest.mark.parametrize("rows", [3, 40])
def test_top_k_on_shapes_of_logits_that_defeat_a_threshold(rows):
    # the chunk's largest are found through a threshold taken from the threads' maxima; these rows make that
    # threshold useless or the gathered set huge (plateaus, sorted rows, nearly everything minus infinity, all large values behind one thread),
    # in chunks that fit the shared memory (3 rows) and in chunks that do not (40 rows)
    from xinfer_b200.sampling import SamplingParams
    vocab = 151936
    rng = np.random.default_rng(rows)
    base = (rng.normal(size=vocab) * 3).astype(np.float32)
    shapes = [
        np.zeros(vocab, dtype=np.float32),                                   # all equal: the lowest indices win
        np.sort(base),                                                        # ascending
        np.sort(base)[::-1].copy(),                                           # descending
        np.where(rng.random(vocab) < 0.05, np.float32(9.0), base),            # a plateau of 7,600 equal maxima
        np.where(rng.random(vocab) < 0.0002, base, np.float32(-np.inf)),      # about 30 finite values
        np.where(np.arange(vocab) % 1024 == 5, base + 30, base),              # every large value in one thread's elements
        np.round(base * 0.05),                                                # zeros of both signs, and little else
    ]
    combos = [(20, 0.95), (1, None), (256, None), (257, 0.9), (None, 0.8), (1000, None), (64, 0.5)]
    logits = np.stack([shapes[r % len(shapes)] for r in range(rows)]).astype(np.float32)
    for shift in range(len(combos) if rows == 3 else 2):
        use = [combos[(r + shift) % len(combos)] for r in range(rows)]
        params = [SamplingParams(temperature=0.8, top_k=k, top_p=p) for k, p in use]
        seeds = list(range(7, 7 + rows))
        got = run(logits, params, seeds, [shift] * rows)
        want = [plain.sample(logits[r], 0.8, top_k=use[r][0] or 0, top_p=use[r][1] if use[r][1] is not None else 1.0,
                             seed=seeds[r], draw=shift) for r in range(rows)]
        assert got == want, (shift, got, want)


@pytest.mark.parametrize("seed", range(3))
def test_random_rows_and_options(seed):
    # random vocabularies, row counts, scales (coarse values, halves of minus infinity) and options per row
    from xinfer_b200.sampling import SamplingParams
    rng = np.random.default_rng(2024 + seed)
    for trial in range(10):
        vocab = int(rng.choice([7, 64, 257, 1000, 4097, 32000, 151936]))
        rows = int(rng.choice([1, 2, 5, 8, 17, 40, 64, 150]))
        rows = max(1, min(rows, int(3e6 // vocab)))
        logits = (rng.normal(size=(rows, vocab)) * float(rng.choice([0.1, 1, 3, 10]))).astype(np.float32)
        if rng.random() < 0.5:
            logits = np.round(logits * 4) / 4
        if rng.random() < 0.2:
            logits[:, : vocab // 2] = -np.inf
        params = [SamplingParams(temperature=float(rng.choice([0.0, 0.3, 0.8, 1.0, 2.0])),
                                 top_k=int(rng.choice([0, 1, 2, 20, 50, 64, 65, 100, 256, 300, 1024, 5000])),
                                 top_p=float(rng.choice([1.0, 0.0, 0.1, 0.5, 0.9, 0.95, 0.999]))) for _ in range(rows)]
        seeds = [int(rng.integers(0, 2 ** 40)) for _ in range(rows)]
        got = run(logits, params, seeds, [trial] * rows)
        want = [plain.sample(logits[r], params[r].temperature, top_k=params[r].top_k, top_p=params[r].top_p, seed=seeds[r], draw=trial)
                for r in range(rows)]
        assert got == want, (trial, vocab, rows, [(r, params[r]) for r in range(rows) if got[r] != want[r]][:3])
