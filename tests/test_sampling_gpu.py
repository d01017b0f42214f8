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
