"""Safetensors by name, one clear error, random-weights mode (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import TINY
from xinfer_b200.config import Qwen3Config
from xinfer_b200.models import model_weight_specs
from xinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, WeightStore, 
                                 write_random_model, write_safetensors)


def test_reader_agrees_with_the_safetensors_package(tmp_path):
    from safetensors.torch import save_file
    tensors = {
        "a.weight": torch.randn(5, 7).to(torch.bfloat16),
        "b.weight": torch.randn(3, 2, 4),
        "c.table": torch.arange(12, dtype=torch.int64).reshape(3, 4),
        "d.half": torch.randn(9).to(torch.float16),
    }
    path = str(tmp_path / "model.safetensors")
    save_file(tensors, path, metadata={"format": "pt"})
    f = SafetensorsFile(path)
    assert set(f.entries) == set(tensors)
    for k, v in tensors.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and tuple(got.shape) == tuple(v.shape)
        assert torch.equal(got, v)
    assert f.metadata["format"] == "pt"


def test_writer_is_read_by_the_safetensors_package(tmp_path):
    from safetensors import safe_open
    tensors = {"x": torch.randn(4, 6).to(torch.bfloat16), "y": torch.randn(10)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, [(k, tuple(v.shape), v.dtype) for k, v in tensors.items()], lambda n: tensors[n])
    with safe_open(path, framework="pt") as f:
        assert set(f.keys()) == set(tensors)
        for k in tensors:
            assert torch.equal(f.get_tensor(k), tensors[k])


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError):
        WeightStore(str(tmp_path / "nowhere"))


def test_dtype_policy(tmp_path):
    from safetensors.torch import save_file
    save_file({"w16": torch.randn(4, 4).to(torch.float16), "wb": torch.randn(4, 4).to(torch.bfloat16),
               "w32": torch.randn(4, 4), "tab": torch.arange(6, dtype=torch.int64)},
              str(tmp_path / "model.safetensors"))
    s = WeightStore(str(tmp_path))
    assert s.get("w16", "cpu", torch.bfloat16).dtype == torch.bfloat16
    assert s.get("wb", "cpu", torch.bfloat16).dtype == torch.bfloat16
    assert s.get("w32", "cpu", torch.bfloat16).dtype == torch.float32   # stored in 32-bit stays so ...
    # ... unless a part asks for it as an operand of the engine's matrix products
    assert s.get("w32", "cpu", torch.bfloat16, operand=True).dtype == torch.bfloat16
    assert s.get("w32", "cpu", torch.float32, operand=True).dtype == torch.float32
    assert s.get("tab", "cpu", torch.bfloat16, operand=True).dtype == torch.int32
    assert s.get("tab", "cpu", torch.bfloat16).dtype == torch.int32      # integer tables as int32
    assert s.get("wb", "cpu", torch.float32).dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file
    raw, seed = TINY["A"]
    write_random_model(str(tmp_path), raw, seed, dtype=torch.float32)
    specs = model_weight_specs(Qwen3Config.from_dict(raw).plan())
    WeightStore(str(tmp_path)).check(specs)  # a fresh folder is complete
    path = str(tmp_path / "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.self_attn.k_norm.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.mlp.extra.weight"] = torch.zeros(2)
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 100)
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        WeightStore(str(tmp_path)).check(specs)
    msg = str(e.value)
    assert e.value.missing == ["model.layers.1.self_attn.k_norm.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert e.value.wrong_shape[0][0] == "model.layers.0.mlp.down_proj.weight"
    for frag in ("missing (2)", "unexpected (1)", "wrong shape (1)", "[64, 100]", "[64, 128]", "k_norm"):
        assert frag in msg


def test_a_spare_head_beside_a_tied_one_is_a_warning_and_an_untied_head_is_required(tmp_path):
    from xinfer_b200.weights import UnexpectedWeightsWarning
    raw, seed = TINY["B"]
    write_random_model(str(tmp_path / "untied"), raw, seed, dtype=torch.bfloat16)
    tied = dict(raw, tie_word_embeddings=True)
    tied_specs = model_weight_specs(Qwen3Config.from_dict(tied).plan())
    store = WeightStore(str(tmp_path / "untied"))
    with pytest.warns(UnexpectedWeightsWarning, match="lm_head.weight"):
        assert store.check(tied_specs) == ["lm_head.weight"]
    assert store.unexpected == ["lm_head.weight"]
    with pytest.raises(WeightError) as e:                      # on request the same is fatal
        store.check(tied_specs, strict=True)
    assert e.value.unexpected == ["lm_head.weight"] and not e.value.missing
    # the other way round: a folder written for a tied head lacks the head an untied model needs
    write_random_model(str(tmp_path / "tied"), tied, seed, dtype=torch.bfloat16)
    with pytest.raises(WeightError) as e:
        WeightStore(str(tmp_path / "tied")).check(model_weight_specs(Qwen3Config.from_dict(raw).plan()))
    assert e.value.missing == ["lm_head.weight"]


def test_random_model_is_seeded_and_order_free(tmp_path):
    from safetensors.torch import load_file
    raw, _ = TINY["C"]
    a = load_file(os.path.join(write_random_model(str(tmp_path / "a"), raw, 7), "model.safetensors"))
    b = load_file(os.path.join(write_random_model(str(tmp_path / "b"), raw, 7), "model.safetensors"))
    c = load_file(os.path.join(write_random_model(str(tmp_path / "c"), raw, 8), "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    # a tensor's values do not depend on which other tensors exist
    fewer = dict(raw, num_hidden_layers=1)
    d = load_file(os.path.join(write_random_model(str(tmp_path / "d"), fewer, 7), "model.safetensors"))
    assert torch.equal(a["model.layers.0.mlp.up_proj.weight"], d["model.layers.0.mlp.up_proj.weight"])
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16
    w = a["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.004
    n = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.1
    assert json.load(open(tmp_path / "a" / "config.json"))["vocab_size"] == raw["vocab_size"]
