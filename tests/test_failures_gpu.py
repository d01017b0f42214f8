"""A step that fails in the middle of generation: its requests end as aborted with the reason,
their pages come back, nothing stays scheduled, and the engine serves the next requests.  Every
failure is made on the host (an exception from the step function, an error word written from the
host); no kernel is made to fault or hang."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import PAGE_SIZE, prompts_for

pytestmark = pytest.mark.gpu

POOL = 64


def engine(folder, dtype, **kw):
    from xinfer_b200 import Engine, EngineConfig
    opts = dict(weight_path=folder, block_size=PAGE_SIZE["A"], num_blocks=POOL, max_num_seqs=3,
                max_num_batched_tokens=256, prefill_chunk_size=256, disable_cuda_graph=True)
    opts.update(kw)
    return Engine(EngineConfig(**opts), dtype)


def whole_again(eng, cfg, w):
    """The engine is as good as new: pool whole, nothing live, and it generates the plain tokens."""
    from xinfer_b200 import SamplingParams
    eng.runner.cache.check_consistent()
    assert eng.runner.cache.free_pages() == POOL
    assert eng.runner.cache.live_requests() == 0
    assert not eng.has_work()
    p = prompts_for("A", [13], seed=9)[0]
    out = eng.generate_sync(SamplingParams(max_tokens=7, ignore_eos=True), [p])[0]
    assert out.error is None and out.finish_reason == "length"
    assert out.decode_output == plain.generate(cfg, w, p, 7)
    eng.runner.cache.check_consistent()
    assert eng.runner.cache.free_pages() == POOL


@pytest.mark.parametrize("run_ahead", [False, True], ids=["step_by_step", "run_ahead"])
def test_an_exception_from_the_step_function_aborts_its_batch_and_the_rest_goes_on(run_ahead, model_folders, monkeypatch):
    """Five requests through three slots; the step function raises once while three of them decode.
    Those three abort with the reason; the two that waited are served afterwards and get the plain
    implementation's tokens."""
    from xinfer_b200 import SamplingParams
    from xinfer_b200.engine.runner import ModelRunner, StepError
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("A", [6, 11, 17, 9, 14], seed=5)
    eng = engine(folder, "f32", disable_run_ahead=not run_ahead)
    real = ModelRunner.step
    calls = {"n": 0}

    def flaky(self, entries, **kw):
        calls["n"] += 1
        if calls["n"] == 5:          # step 1 prefills three prompts; by step 5 they decode
            raise StepError("injected on the host")
        return real(self, entries, **kw)

    monkeypatch.setattr(ModelRunner, "step", flaky)
    outs = eng.generate_sync(SamplingParams(max_tokens=12, ignore_eos=True), prompts)
    assert eng.stats["failed_steps"] == 1
    aborted = [o for o in outs if o.finish_reason == "abort"]
    assert [o.seq_id for o in aborted] == [0, 1, 2]
    for o in aborted:
        assert "StepError: injected on the host" in o.error
        assert 1 <= o.decoded_length < 12      # what they had decoded is kept
        p = prompts[o.seq_id]
        assert o.decode_output == plain.generate(cfg, w, p, 12)[: o.decoded_length]
    for o in outs[3:]:
        assert o.error is None and o.finish_reason == "length"
        assert o.decode_output == plain.generate(cfg, w, prompts[o.seq_id], 12)
    monkeypatch.setattr(ModelRunner, "step", real)
    whole_again(eng, cfg, w)


@pytest.mark.parametrize("dtype,graphs,run_ahead", [("f32", False, False), ("bf16", False, True), ("bf16", True, True)],
                         ids=["f32", "bf16_run_ahead", "bf16_graphs_run_ahead"])
def test_an_error_word_from_the_device_aborts_the_batches_in_flight(dtype, graphs, run_ahead, model_folders):
    """The device error word is set from the host (as a kernel that met a bad page id would set it)
    while requests decode - with a second batch already queued behind the running one where the
    next step is decided ahead.  Both batches' requests abort, the word is cleared, the pool is whole."""
    from xinfer_b200 import SamplingParams, kernels
    store = torch.float32 if dtype == "f32" else torch.bfloat16
    folder = model_folders("A", store)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("A", [8, 15, 21], seed=6)
    eng = engine(folder, dtype, disable_run_ahead=not run_ahead, disable_cuda_graph=not graphs)
    ids = [eng.add_request(p, SamplingParams(max_tokens=30, ignore_eos=True)) for p in prompts]
    for _ in range(6):
        eng.step()
    assert all(i in eng._live for i in ids)
    assert (eng._flight is not None) == run_ahead          # a batch is queued behind the running one
    eng.runner.err.fill_(kernels.ERR_BAD_PAGE)
    while any(i in eng._live for i in ids):
        eng.step()
    assert eng.stats["failed_steps"] == 1
    for i in ids:
        out = eng._done.pop(i)
        assert out.finish_reason == "abort" and "outside the page pool" in out.error
        assert out.decoded_length >= 4
    assert int(eng.runner.err.item()) == 0
    whole_again(eng, cfg, w)


def test_a_stream_reports_the_failure(model_folders, monkeypatch):
    from xinfer_b200 import SamplingParams
    from xinfer_b200.engine.runner import ModelRunner, StepError
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    eng = engine(folder, "f32")
    real = ModelRunner.step
    calls = {"n": 0}

    def flaky(self, entries, **kw):
        calls["n"] += 1
        if calls["n"] == 4:
            raise StepError("injected on the host")
        return real(self, entries, **kw)

    monkeypatch.setattr(ModelRunner, "step", flaky)
    p = prompts_for("A", [10], seed=2)[0]
    _, _, items = eng.generate_stream(SamplingParams(max_tokens=10, ignore_eos=True), p)
    items = list(items)
    assert items[-1].datatype == "ERROR" and "injected" in items[-1].data
    toks = [i.data for i in items if i.datatype == "TOKEN_ID"]
    assert toks and toks == plain.generate(cfg, w, p, 10)[: len(toks)]
    monkeypatch.setattr(ModelRunner, "step", real)
    whole_again(eng, cfg, w)
