"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from helpers import TINY
from xinfer_b200.config import (ConfigError, EngineConfig, Qwen3Config, config_from_dict,
                                known_architectures, load_config, register_architecture,
                                unregister_architecture)
from xinfer_b200.config.plan import LayerRun


def test_reads_every_key_from_config_json():
    for name, (raw, _) in TINY.items():
        entry, cfg = config_from_dict(raw)
        assert entry.name == "Qwen3ForCausalLM"
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps",
                    "rope_theta", "max_position_embeddings", "tie_word_embeddings", "sliding_window"):
            assert getattr(cfg, key) == raw[key], (name, key)


def test_defaults():
    raw = dict(TINY["A"][0])
    del raw["head_dim"], raw["rope_theta"], raw["tie_word_embeddings"], raw["sliding_window"]
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert cfg.rope_theta == 10000.0
    assert cfg.tie_word_embeddings is False
    assert cfg.sliding_window is None
    assert cfg.eos_token_id == (255,)
    assert Qwen3Config.from_dict(TINY["B"][0]).eos_token_id == (3, 5)


@pytest.mark.parametrize("change, fragment", [
    (dict(vocab_size=None), "vocab_size"),
    (dict(num_attention_heads=5), "multiple of num_key_value_heads"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(sliding_window=-3), "sliding_window"),
    (dict(hidden_size="64"), "hidden_size"),
    (dict(head_dim=15), "head_dim"),
    (dict(eos_token_id="x"), "eos_token_id"),
])
def test_errors_name_the_key(change, fragment):
    raw = dict(TINY["A"][0])
    raw.update(change)
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    assert fragment in str(e.value)


def test_missing_keys_are_listed_together():
    raw = dict(TINY["A"][0])
    del raw["vocab_size"], raw["rms_norm_eps"]
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    assert "vocab_size" in str(e.value) and "rms_norm_eps" in str(e.value)


def test_registry_unknown_and_malformed():
    raw = dict(TINY["A"][0], architectures=["NoSuchModel"])
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert "NoSuchModel" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict(dict(TINY["A"][0], architectures=["a", "b"]))
    with pytest.raises(ConfigError):
        config_from_dict({k: v for k, v in TINY["A"][0].items() if k != "architectures"})


def test_register_another_architecture():
    def plan_of(cfg):
        return Qwen3Config.from_dict(cfg).plan()
    register_architecture("ToyForTest", lambda raw: dict(raw), plan_of)
    try:
        assert "ToyForTest" in known_architectures()
        with pytest.raises(ValueError):
            register_architecture("ToyForTest", lambda raw: raw, plan_of)
        entry, cfg = config_from_dict(dict(TINY["A"][0], architectures=["ToyForTest"]))
        assert entry.plan_of(cfg).vocab_size == 256
    finally:
        unregister_architecture("ToyForTest")
    assert "ToyForTest" not in known_architectures()


def test_plan_carries_every_constant():
    for name, (raw, _) in TINY.items():
        cfg = Qwen3Config.from_dict(raw)
        plan = cfg.plan()
        assert len(plan.blocks) == raw["num_hidden_layers"] == len(plan.runs)
        assert [r.block for r in plan.runs] == list(range(raw["num_hidden_layers"]))
        b = plan.blocks[-1]
        assert b.mixer.num_heads == raw["num_attention_heads"] and b.mixer.num_kv_heads == raw["num_key_value_heads"]
        assert b.mixer.head_dim == raw["head_dim"] and b.mixer.window == raw["sliding_window"]
        assert b.mixer.scale == pytest.approx(raw["head_dim"] ** -0.5)
        assert b.mixer.rope.theta == raw["rope_theta"] and b.mixer.rope.max_positions == raw["max_position_embeddings"]
        assert b.mixer.qk_norm and b.mixer.qk_norm_eps == raw["rms_norm_eps"]
        assert [n.eps for n in b.norms()] == [raw["rms_norm_eps"]] * 2 and plan.final_norm.eps == raw["rms_norm_eps"]
        assert [o.op for o in b.program] == ["norm", "mixer", "add", "norm", "feed_forward", "add"]
        assert b.feed_forward.intermediate == raw["intermediate_size"]
        assert (plan.head_name is None) == bool(raw["tie_word_embeddings"])


def test_plan_validation_of_the_run_list():
    plan = Qwen3Config.from_dict(TINY["A"][0]).plan()
    import dataclasses
    ok = dataclasses.replace(plan, runs=(LayerRun(0), LayerRun(1), LayerRun(1), LayerRun(0, cache_from=0)))
    ok.validate()
    for bad in ((LayerRun(0), LayerRun(5)), (LayerRun(0, cache_from=0),), (LayerRun(0), LayerRun(1, cache_from=1)),
                (LayerRun(0), LayerRun(1, cache_from=0), LayerRun(0, cache_from=1))):
        with pytest.raises(ValueError):
            dataclasses.replace(plan, runs=bad).validate()


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"][0]))
    entry, cfg = load_config(str(tmp_path))
    assert cfg.num_key_value_heads == 1 and cfg.to_dict()["model_type"] == "qwen3"


def test_engine_config_validation():
    EngineConfig(weight_path="x").validate()
    assert EngineConfig(model_id="m").model_dir() == "m"
    with pytest.raises(ValueError):
        EngineConfig().model_dir()
    for bad in (dict(block_size=0), dict(max_num_seqs=-1), dict(kv_fraction=0.0), dict(num_blocks=0)):
        with pytest.raises(ValueError):
            EngineConfig(weight_path="x", **bad).validate()


def test_the_longest_sequence_may_not_exceed_the_position_tables():
    from xinfer_b200.engine.runner import resolve_max_model_len
    assert resolve_max_model_len(None, 512) == 512
    assert resolve_max_model_len(200, 512) == 200
    assert resolve_max_model_len(512, 512) == 512
    with pytest.raises(ConfigError, match="max_position_embeddings 512"):
        resolve_max_model_len(513, 512)
    with pytest.raises(ConfigError, match="positive"):
        resolve_max_model_len(0, 512)


def test_a_block_is_a_program_and_bad_programs_are_refused():
    from xinfer_b200.config import BlockOp, BlockSpec, FeedForwardSpec, NormSpec, pre_norm_block
    from xinfer_b200.config.plan import PartSpec
    n = NormSpec(kind="rmsnorm", dim=8)
    m, f = PartSpec(kind="some_mixer"), FeedForwardSpec(kind="swiglu", hidden=8, intermediate=16)
    b = pre_norm_block("l.", n, m, n, f)
    b.validate()
    assert b.mixer is m and b.feed_forward is f and len(b.norms()) == 2
    assert [o.name for o in b.program if o.spec is not None] == ["input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp."]
    # no feed-forward, no mixer: both are fine
    BlockSpec("l.", (BlockOp("norm", "x", "h", n, "n."), BlockOp("mixer", "h", "a", m, "m."), BlockOp("add", "a", "x"))).validate()
    only_ffn = BlockSpec("l.", (BlockOp("feed_forward", "x", "f", f, "f."), BlockOp("add", "f", "x")))
    only_ffn.validate()
    assert only_ffn.mixer is None
    bad = [
        (BlockOp("norm", "y", "h", n, "n."),),                                        # reads what nothing produced
        (BlockOp("add", "x", "y"),),                                                  # adds into what nothing produced
        (BlockOp("add", "x", "x"),),                                                  # a value to itself
        (BlockOp("mixer", "x", "x", m, "m."),),                                       # a part over its own input
        (BlockOp("norm", "x", "h", None, "n."),),                                     # no spec
        (BlockOp("gate", "x", "h", n, "n."),),                                        # unknown operation
        (BlockOp("mixer", "x", "a", m, "m1."), BlockOp("mixer", "x", "b", m, "m2.")),   # two mixers
    ]
    for prog in bad:
        with pytest.raises(ValueError):
            BlockSpec("l.", prog).validate()


def test_nvtx_ranges_follow_the_flag():
    from xinfer_b200 import tracing
    calls = []
    was = tracing.ENABLED
    try:
        tracing.enable(True, push=lambda name: calls.append(("push", name)), pop=lambda: calls.append(("pop",)))
        tracing.push("decode step")
        tracing.pop()
        assert calls == [("push", "decode step"), ("pop",)]
        tracing.enable(False)
        tracing.push("nothing")
        tracing.pop()
        assert len(calls) == 2 and not tracing.ENABLED
    finally:
        tracing.enable(was)
    assert tracing.step_kind([1, 1, 1]) == "decode" and tracing.step_kind([5, 9]) == "prefill"
    assert tracing.step_kind([1, 7]) == "mixed"


def test_generation_config_reads_merges_and_fills(tmp_path):
    import json
    from xinfer_b200 import GenerationConfig, SamplingParams
    from xinfer_b200.config.generation import join_eos
    assert GenerationConfig.load(str(tmp_path)) is None                      # a folder without the file
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"temperature": 0.6, "top_k": 20, "top_p": 0.95, "eos_token_id": [7, 3], "do_sample": True, "bos_token_id": 1}))
    g = GenerationConfig.load(str(tmp_path))
    assert (g.temperature, g.top_k, g.top_p, g.frequency_penalty, g.bos_token_id, g.eos_token_id) == (0.6, 20, 0.95, None, 1, (7, 3))
    # the engine's own options come first, field by field
    m = GenerationConfig(temperature=0.0, presence_penalty=1.5).over(g)
    assert (m.temperature, m.top_k, m.top_p, m.presence_penalty, m.eos_token_id) == (0.0, 20, 0.95, 1.5, (7, 3))
    assert GenerationConfig(top_k=5).over(None).top_k == 5
    # a request keeps what it sets, and is not changed in place
    p = SamplingParams(temperature=1.0, max_tokens=9)
    f = g.fill(p)
    assert (f.temperature, f.top_k, f.top_p, f.max_tokens) == (1.0, 20, 0.95, 9) and p.top_k is None
    assert GenerationConfig().fill(p) is p
    # EOS ids: config.json's first, then what only the generation config names
    assert join_eos((3,), g) == (3, 7) and join_eos((), g) == (7, 3) and join_eos((4,), None) == (4,)
    for bad in ({"temperature": "hot"}, {"top_k": 2.5}, {"eos_token_id": "x"}, {"top_p": True}):
        (tmp_path / "generation_config.json").write_text(json.dumps(bad))
        with pytest.raises(ConfigError):
            GenerationConfig.load(str(tmp_path))
    (tmp_path / "generation_config.json").write_text("{ not json")
    with pytest.raises(ConfigError):
        GenerationConfig.load(str(tmp_path))


def test_command_line_refuses_what_the_engine_does_not_do():
    from xinfer_b200.cli import main
    for argv, word in ((["--m", "x", "--cpu"], "no CPU path"), (["--m", "x", "--d", "0,1"], "one GPU"),
                       (["--m", "x", "--d", "gpu"], "one GPU"), (["--m", "x", "--w", "y"], "either"), ([], "required")):
        with pytest.raises(SystemExit) as e:
            main(argv)
        assert word in str(e.value)


def test_engine_config_takes_the_references_options_and_refuses_what_is_not_built():
    # the options of the reference's Python example, none of them asking for an unbuilt feature
    ec = EngineConfig(model_id=None, weight_path="/m", weight_file=None, max_num_seqs=2, max_model_len=512, max_tokens=64, isq=None,
                      device_ids=[0], generation_cfg=None, disable_prefix_cache=True, prefix_cache_max_tokens=None,
                      kvcache_dtype=None, server_mode=False, cpu_mem_fold=None, kv_fraction=0.5, disable_reasoning=True,
                      disable_cuda_graph=False, prefill_chunk_size=8192)
    ec.validate()
    assert ec.device == "cuda:0"
    for kw, word in ((dict(isq="q4k"), "isq"), (dict(kvcache_dtype="fp8"), "kvcache_dtype"), (dict(device_ids=[0, 1]), "device_ids"),
                     (dict(num_shards=2), "num_shards"), (dict(weight_file="m.gguf"), "weight_file"), (dict(server_mode=True), "server_mode"),
                     (dict(cpu_mem_fold=0.5), "cpu_mem_fold"), (dict(mtp_num_speculative_tokens=2), "speculative")):
        with pytest.raises(ValueError, match=word):
            EngineConfig(weight_path="/m", **kw).validate()
