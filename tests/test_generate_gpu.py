"""Generation through the Python entry point against the plain implementation."""
import pytest
import torch

import plain_qwen3 as plain
from helpers import PAGE_SIZE, TINY, prompts_for

TINY_A = TINY["A"][0]

pytestmark = pytest.mark.gpu


def engine(folder, dtype, name, **kw):
    from xinfer_b200 import Engine, EngineConfig
    opts = dict(weight_path=folder, block_size=PAGE_SIZE[name], num_blocks=64, max_num_seqs=4,
                max_num_batched_tokens=256, prefill_chunk_size=256, disable_cuda_graph=True)
    opts.update(kw)
    return Engine(EngineConfig(**opts), dtype)


def test_greedy_float32_equals_plain(model_folders):
    # tiny configuration A: three prompts of 5 / 11 / 17 tokens, whole, 8 greedy steps each
    from xinfer_b200 import SamplingParams
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("A", [5, 11, 17])
    outs = engine(folder, "f32", "A").generate_sync(SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True), prompts)
    for p, o in zip(prompts, outs):
        assert o.decode_output == plain.generate(cfg, w, p, 8)
        assert (o.prompt_length, o.decoded_length, o.finish_reason) == (len(p), 8, "length")
        assert o.prompt_start_time <= o.decode_start_time <= o.decode_finish_time


def test_portions_of_six_and_temperature_sampling_equal_plain(model_folders):
    # tiny configuration B: prompts of 1 / 7 / 23 / 40 tokens in portions of 6, temperature 0.8, 10 steps
    from xinfer_b200 import SamplingParams
    folder = model_folders("B", torch.float32)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("B", [1, 7, 23, 40])
    eng = engine(folder, "f32", "B", prefill_chunk_size=6, max_num_batched_tokens=16)
    params = [SamplingParams(temperature=0.8, max_tokens=10, ignore_eos=True, seed=50 + i) for i in range(4)]
    outs = eng.generate_sync(params, prompts)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert o.decode_output == plain.generate(cfg, w, p, 10, temperature=0.8, seed=50 + i)
    assert eng.stats["steps"] > 10 + 40 // 6


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "cuda_graph"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_bfloat16_greedy_follows_the_plain_logits(name, graphs, model_folders):
    """bfloat16 may flip a near-tie, so each generated token is checked against the plain logits
    of the sequence the engine actually produced: it must be the best token up to the drift.
    Decode steps launched kernel by kernel, and replayed from CUDA graphs."""
    from xinfer_b200 import SamplingParams
    folder = model_folders(name, torch.bfloat16)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for(name, [3, 30, 61])
    eng = engine(folder, "bf16", name, disable_cuda_graph=not graphs)
    outs = eng.generate_sync(SamplingParams(max_tokens=40, ignore_eos=True), prompts)
    assert eng.runner.last_used_graph == graphs
    for p, o in zip(prompts, outs):
        seq = p + o.decode_output
        ref = plain.forward(cfg, w, seq)
        drift = 3.0 * (plain.forward(cfg, w, seq, round_to=torch.bfloat16) - ref).abs().max().item()
        for i, tok in enumerate(o.decode_output):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - 2 * drift, (i, tok)


def test_long_decoding_and_first_tokens(model_folders):
    from xinfer_b200 import SamplingParams
    folder = model_folders("C", torch.float32)     # window 37: pages behind the window are given back
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("C", [1, 2, 9])
    eng = engine(folder, "f32", "C", num_blocks=12)  # 192 tokens of pages for 3 requests growing to ~300 each
    outs = eng.generate_sync(SamplingParams(max_tokens=300, ignore_eos=True), prompts)
    for p, o in zip(prompts, outs):
        assert o.decoded_length == 300
        seq = p + o.decode_output
        ref = plain.forward(cfg, w, seq)
        for i, tok in enumerate(o.decode_output):   # teacher-forced: each token is the plain argmax
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - 1e-5, (i, tok)
    assert eng.stats["preemptions"] == 0
    eng.runner.cache.check_consistent()
    assert eng.runner.cache.live_requests() == 0


def test_top_k_top_p_and_penalties_equal_plain(model_folders):
    from xinfer_b200 import SamplingParams
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts_for("A", [12])[0]
    eng = engine(folder, "f32", "A")
    for kw in (dict(top_k=5), dict(top_p=0.7), dict(top_k=12, top_p=0.8)):
        o = eng.generate_sync(SamplingParams(temperature=1.1, max_tokens=12, ignore_eos=True, seed=9, **kw), [p])[0]
        assert o.decode_output == plain.generate(cfg, w, p, 12, temperature=1.1, seed=9,
                                                 top_k=kw.get("top_k", 0), top_p=kw.get("top_p", 1.0)), kw
    o = eng.generate_sync(SamplingParams(temperature=0.9, max_tokens=20, ignore_eos=True, seed=4,
                                         frequency_penalty=1.5, presence_penalty=0.5), [p])[0]
    ids = list(p)
    for n in range(20):
        logits = plain.apply_penalties(plain.forward(cfg, w, ids)[-1].numpy(), ids[-128:], 1.5, 0.5)
        ids.append(plain.sample(logits, 0.9, seed=4, draw=n))
    assert o.decode_output == ids[len(p):]


def test_eos_stop_tokens_and_stream(model_folders):
    from xinfer_b200 import SamplingParams
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts_for("A", [10])[0]
    free = plain.generate(cfg, w, p, 12)
    eng = engine(folder, "f32", "A")
    stop = free[5]
    o = eng.generate_sync(SamplingParams(max_tokens=12, ignore_eos=True, stop_token_ids=[stop]), [p])[0]
    assert o.decode_output == free[: free.index(stop)] and o.finish_reason == "stop"
    seq_id, plen, stream = eng.generate_stream(SamplingParams(max_tokens=12, ignore_eos=True), p)
    items = list(stream)
    assert plen == 10 and [i.data for i in items if i.datatype == "TOKEN_ID"] == free
    assert items[-1].datatype == "DONE" and items[-1].data[:3] == (seq_id, 10, 12)
    assert eng.get_available_kv_tokens() == 64 * 16 and eng.get_num_cached_tokens() == 0


def test_scarce_pages_preempt_and_still_give_the_same_tokens(model_folders):
    from xinfer_b200 import SamplingParams
    folder = model_folders("B", torch.float32)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("B", [30, 26, 22, 18], seed=3)
    sp = [SamplingParams(temperature=0.7, max_tokens=40, ignore_eos=True, seed=i) for i in range(4)]
    roomy = engine(folder, "f32", "B", num_blocks=64).generate_sync(sp, prompts)
    tight_engine = engine(folder, "f32", "B", num_blocks=20)     # 160 tokens for 4 requests that grow to ~260
    tight = tight_engine.generate_sync(sp, prompts)
    assert tight_engine.stats["preemptions"] > 0
    for a, b, p, s in zip(roomy, tight, prompts, sp):
        assert a.decode_output == b.decode_output
        assert a.decode_output == plain.generate(cfg, w, p, 40, temperature=0.7, seed=s.seed)
    tight_engine.runner.cache.check_consistent()
    assert tight_engine.runner.cache.free_pages() == 20


def test_bad_requests_are_refused(model_folders):
    from xinfer_b200 import SamplingParams
    from xinfer_b200.engine.scheduler import SchedulerError
    folder = model_folders("A", torch.float32)
    eng = engine(folder, "f32", "A", num_blocks=4, max_model_len=128)
    with pytest.raises(ValueError):
        eng.generate_sync(SamplingParams(max_tokens=2), [[1, 2, 999]])
    with pytest.raises(SchedulerError, match="never fit"):
        eng.generate_sync(SamplingParams(max_tokens=60), [[1] * 30])
    with pytest.raises(SchedulerError, match="too long"):
        eng.generate_sync(SamplingParams(max_tokens=2), [[1] * 128])
    assert eng.generate_sync(SamplingParams(max_tokens=3, ignore_eos=True), [[1, 2, 3]])[0].decoded_length == 3


def test_command_line(model_folders, capsys):
    from xinfer_b200.cli import main
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    assert main(["--m", folder, "--dtype", "f32", "--prompts", "5,6,7|9,10", "--max-tokens", "4", "--ignore-eos",
                 "--disable-cuda-graph", "--num-blocks", "16", "--d", "0"]) == 0
    out = capsys.readouterr().out
    want = ",".join(str(t) for t in plain.generate(cfg, w, [5, 6, 7], 4))
    assert want in out and "Prompt tokens: 5" in out and "Decoded tokens: 8" in out
    # the sampling flags are the engine's defaults for requests that set nothing (top-k 1: the best token whatever the temperature)
    assert main(["--m", folder, "--dtype", "f32", "--prompts", "5,6,7", "--max-tokens", "4", "--ignore-eos", "--num-blocks", "16",
                 "--temperature", "3.0", "--top-k", "1", "--seed", "5"]) == 0
    assert want in capsys.readouterr().out


@pytest.mark.parametrize("dtype,graphs", [("f32", False), ("bf16", True), ("bf16", False)])
def test_deciding_the_next_step_ahead_changes_no_token(dtype, graphs, model_folders):
    """The same requests with and without the next decode step being queued while the current one
    runs: stop tokens found late, requests ending by length at different steps, sampling with
    temperature, requests arriving while others decode."""
    from xinfer_b200 import SamplingParams
    store = torch.float32 if dtype == "f32" else torch.bfloat16
    folder = model_folders("B", store)       # configuration B stops on tokens 3 and 5
    prompts = prompts_for("B", [4, 19, 33, 7, 12, 26], seed=3)
    params = [SamplingParams(temperature=0.0 if i % 2 else 0.9, top_k=0 if i % 3 else 20, max_tokens=5 + 9 * i,
                             ignore_eos=(i == 1), seed=7 + i) for i in range(len(prompts))]
    runs = []
    for off in (True, False):
        eng = engine(folder, dtype, "B", disable_run_ahead=off, disable_cuda_graph=not graphs, max_num_seqs=3)
        outs = eng.generate_sync(params, prompts)     # six requests through three slots
        runs.append([(o.decode_output, o.finish_reason) for o in outs])
        assert (eng.stats["steps_decided_ahead"] > 10) == (not off)
        assert not eng.has_work()
        eng.runner.cache.check_consistent()
        assert eng.runner.cache.live_requests() == 0
    assert runs[0] == runs[1]
    assert {r for _, r in runs[0]} >= {"length"}


def test_cache_sized_from_free_memory_and_the_command_line(model_folders, tmp_path, capsys):
    """num_blocks unset: the pool is sized from free device memory x kv_fraction, capped by what
    max_num_seqs requests of max_model_len tokens can hold; the command line prints what the
    Python entry point returns."""
    from xinfer_b200 import SamplingParams
    from xinfer_b200 import cli
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    eng = engine(folder, "f32", "A", num_blocks=None, kv_fraction=0.01, max_num_seqs=2, max_model_len=200)
    assert eng.runner.num_blocks == 2 * ((200 + 15) // 16)          # the cap, far below 1 % of a B200
    assert eng.get_available_kv_tokens() == eng.runner.num_blocks * 16
    p = prompts_for("A", [9])[0]
    want = plain.generate(cfg, w, p, 6)
    assert eng.generate_sync(SamplingParams(max_tokens=6, ignore_eos=True), [p])[0].decode_output == want
    rc = cli.main(["--m", folder, "--dtype", "f32", "--prompts", ",".join(map(str, p)), "--max-tokens", "6", "--ignore-eos",
                   "--kv-fraction", "0.01", "--max-model-len", "200"])
    out = capsys.readouterr().out
    assert rc == 0 and ",".join(map(str, want)) in out and "Prompt tokens: 9" in out


def test_graphs_follow_the_context_past_a_table_width(tmp_path):
    """Decode graphs are captured per block-table width (64 pages, then 128, ...): a request decodes
    across the first width while the next step is always queued ahead; every token must still be
    the plain implementation's best token up to the bfloat16 drift."""
    from helpers import sharpen
    from xinfer_b200 import SamplingParams
    from xinfer_b200.weights import write_random_model
    cfg = dict(TINY_A, max_position_embeddings=2048)
    folder = write_random_model(str(tmp_path / "m"), cfg, 4, dtype=torch.bfloat16, override=sharpen)
    cfg, w = plain.load_folder(folder)
    prompts = prompts_for("A", [9, 300])
    eng = engine(folder, "bf16", "A", block_size=8, num_blocks=200, disable_cuda_graph=False, max_model_len=1200)
    outs = eng.generate_sync(SamplingParams(max_tokens=560, ignore_eos=True), prompts)   # 569 and 860 tokens: past 64 pages of 8
    assert len(eng.runner._graphs) >= 2 and eng.stats["steps_decided_ahead"] > 500
    for p, o in zip(prompts, outs):
        assert o.decoded_length == 560
        seq = p + o.decode_output
        ref = plain.forward(cfg, w, seq)
        drift = 3.0 * (plain.forward(cfg, w, seq, round_to=torch.bfloat16) - ref).abs().max().item()
        for i, tok in enumerate(o.decode_output):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - 2 * drift, (i, tok)
    eng.runner.cache.check_consistent()


def test_a_checkpoint_stored_in_float32_runs_a_bfloat16_engine_on_bfloat16_weights(model_folders):
    """Projection, embedding and head matrices take the engine's dtype at load whatever the file
    holds (norm weights stay float32): a decode step then runs on the tcgen05 product, not on the
    float32 FMA product, and the logits are the plain implementation's up to the bfloat16 drift."""
    from xinfer_b200 import kernels
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    r = ModelRunner(folder, "bfloat16", block_size=16, num_blocks=16, max_num_seqs=2)
    block = r.model.blocks[0]
    assert block.mixer.w_qkv.dtype == torch.bfloat16 and block.mixer.w_o.dtype == torch.bfloat16
    assert block.mixer.q_norm.dtype == torch.float32
    assert r.model.embed.dtype == torch.bfloat16 and r.model.final_norm.weight.dtype == torch.float32
    ffn = [p for p in block.all_parts() if p.kind == "swiglu"][0]
    assert ffn.w_gate_up.dtype == torch.bfloat16 and ffn.w_down.dtype == torch.bfloat16
    p = prompts_for("A", [40])[0]
    slot = r.open_request()
    got = [r.step([StepInput(slot, p[:30], range(30))]).float().cpu().clone()]
    before = kernels.launch_counts()
    for j in range(30, 40):
        got.append(r.step([StepInput(slot, p[j:j + 1], [0])]).float().cpu().clone())
    r.check_errors()
    after = kernels.launch_counts()
    assert after.get("gemm_skinny_tc", 0) - before.get("gemm_skinny_tc", 0) >= 10 * (4 * 2 + 1)
    assert after.get("gemm_plain", 0) == before.get("gemm_plain", 0)
    # the engine's weights are the file's rounded to bfloat16: the oracle gets the same
    wb = {k: (v.to(torch.bfloat16).float() if not k.endswith("norm.weight") and "layernorm" not in k else v) for k, v in w.items()}
    ref = plain.forward(cfg, wb, p)
    tol = 3.0 * (plain.forward(cfg, wb, p, round_to=torch.bfloat16) - ref).abs().max().item()
    assert (torch.cat(got) - ref).abs().max().item() <= tol


def test_scarce_pages_under_bfloat16_graphs_and_steps_decided_ahead(model_folders):
    """Preemption while the next decode step is already queued on the device, with decode steps
    replayed from CUDA graphs: the tight pool must give the tokens of the roomy one, and be whole after."""
    from xinfer_b200 import SamplingParams
    folder = model_folders("B", torch.bfloat16)
    prompts = prompts_for("B", [30, 26, 22, 18], seed=3)
    sp = [SamplingParams(temperature=0.7, max_tokens=40, ignore_eos=True, seed=i) for i in range(4)]
    opts = dict(disable_cuda_graph=False, disable_run_ahead=False)
    roomy_engine = engine(folder, "bf16", "B", num_blocks=64, **opts)
    roomy = roomy_engine.generate_sync(sp, prompts)
    assert roomy_engine.stats["preemptions"] == 0 and roomy_engine.stats["steps_decided_ahead"] > 20
    tight_engine = engine(folder, "bf16", "B", num_blocks=20, **opts)     # 160 tokens for 4 requests that grow to ~260
    tight = tight_engine.generate_sync(sp, prompts)
    assert tight_engine.stats["preemptions"] > 0 and tight_engine.stats["steps_decided_ahead"] > 5
    assert tight_engine.runner.last_used_graph
    for a, b in zip(roomy, tight):
        assert a.decode_output == b.decode_output and b.finish_reason == "length"
    tight_engine.runner.cache.check_consistent()
    assert tight_engine.runner.cache.free_pages() == 20 and tight_engine.runner.cache.live_requests() == 0


def test_logits_do_not_change_precision_with_the_number_of_rows():
    """Up to 32 wanted rows the head runs on the engine's tcgen05 product, above on the library's; both
    write float32 accumulators.  The same row's logits at 32 and at 33 rows must agree to float32
    accumulation order, far below the spacing of bfloat16 (which would make ties and move a greedy token)."""
    from xinfer_b200.parts.linear import linear
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    y = (torch.randn(33, 4096, generator=g) * 1.0).to(torch.bfloat16).to(dev)
    head = (torch.randn(5003, 4096, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    a = torch.empty(32, 5003, dtype=torch.float32, device=dev)
    b = torch.empty(33, 5003, dtype=torch.float32, device=dev)
    linear(a, y[:32].contiguous(), head, err)
    linear(b, y, head, err)
    assert int(err) == 0
    ref = y.double() @ head.double().t()
    assert (a.double() - ref[:32]).abs().max().item() < 2e-4 and (b.double() - ref).abs().max().item() < 2e-4
    assert (a - b[:32]).abs().max().item() < 2e-4       # bfloat16 values of this size are 0.016 apart
    # not values of bfloat16: the low 16 bits of the float32 words are in use in both
    for t in (a, b):
        assert (t.view(torch.int32) & 0xFFFF).ne(0).float().mean().item() > 0.9


def test_a_stream_can_be_cancelled_and_stop_sequences_end_a_request(model_folders):
    from xinfer_b200 import SamplingParams
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts_for("A", [12], seed=4)[0]
    free = plain.generate(cfg, w, p, 14)
    eng = engine(folder, "f32", "A")
    # a stream that is cancelled after five tokens: what it had stays, its pages come back, the engine goes on
    seq_id, plen, stream = eng.generate_stream(SamplingParams(max_tokens=14, ignore_eos=True), p)
    assert (stream.seq_id, stream.prompt_length, stream.finished, stream.cancelled) == (seq_id, 12, False, False)
    got = []
    for item in stream:
        if item.datatype == "TOKEN_ID":
            got.append(item.data)
            if len(got) == 5:
                stream.cancel()
        else:
            assert item.datatype == "DONE" and item.data[0] == seq_id
    assert stream.finished and stream.cancelled
    assert 5 <= len(got) <= 7 and got == free[: len(got)]      # at most the tokens of steps already queued come after
    assert eng.runner.cache.live_requests() == 0 and eng.runner.cache.free_pages() == 64 and not eng.has_work()
    # a stop sequence of two ids: the request ends when the generated tokens end with it; its last token stays out
    stop = free[6:8]
    o = eng.generate_sync(SamplingParams(max_tokens=14, ignore_eos=True, stop_token_ids=[[free[2], (free[2] + 1) % 256], stop]), [p])[0]
    first = next(i for i in range(1, 14) if free[i - 1:i + 1] == stop)
    assert o.finish_reason == "stop" and o.decode_output == free[:first]


def test_generation_config_of_the_folder_and_of_the_engine(model_folders, tmp_path):
    import json
    import shutil
    from xinfer_b200 import GenerationConfig, SamplingParams
    src = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(src)
    p = prompts_for("A", [9], seed=11)[0]
    free = plain.generate(cfg, w, p, 12)
    folder = str(tmp_path / "with_generation_config")
    shutil.copytree(src, folder)
    stop_at = next(i for i in range(3, 12) if free[i] not in free[:i])      # a token that generation meets there first
    with open(folder + "/generation_config.json", "w") as f:
        json.dump({"temperature": 5.0, "top_k": 1, "eos_token_id": [free[stop_at]]}, f)
    eng = engine(folder, "f32", "A")
    assert eng.eos_token_ids[-1] == free[stop_at] and eng.generation_cfg.top_k == 1
    # a request that sets nothing takes the folder's options: the one most likely token at any temperature,
    # until the folder's extra EOS id comes (it stays out of the output)
    o = eng.generate_sync(SamplingParams(max_tokens=12), [p])[0]
    assert o.decode_output == free[:stop_at] and o.finish_reason == "stop"
    o = eng.generate_sync(SamplingParams(max_tokens=12, ignore_eos=True), [p])[0]
    assert o.decode_output == free
    # the engine's own options come before the folder's: top-k off, so temperature 5 draws from nearly all tokens
    eng2 = engine(folder, "f32", "A", generation_cfg=GenerationConfig(top_k=0))
    assert (eng2.generation_cfg.temperature, eng2.generation_cfg.top_k) == (5.0, 0)
    o = eng2.generate_sync(SamplingParams(max_tokens=12, ignore_eos=True, seed=3), [p])[0]
    assert o.decode_output != free
    # and a request's own options before both
    o = eng2.generate_sync(SamplingParams(max_tokens=12, ignore_eos=True, temperature=0.0), [p])[0]
    assert o.decode_output == free
