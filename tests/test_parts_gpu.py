"""Each part of a block alone on the GPU against the plain implementation's function for it, at
sizes of their own, and the arrangement of layer runs (a block named twice, a run that reads
another run's cache)."""
import dataclasses

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class FakeStore:
    """Hands the parts tensors from a dict, with the loader's dtype rules."""

    def __init__(self, tensors):
        self.tensors = tensors

    def get(self, name, device, compute_dtype, operand=False):
        t = self.tensors[name]
        if compute_dtype == torch.float32 or (t.dtype == torch.float32 and not operand):
            return t.to(device).float().contiguous()
        return t.to(device).to(torch.bfloat16).contiguous()


def context(entries, dtype, page=8, pages=64, window=None, vocab=100):
    """A cache manager, an assembler and the step context for entries [(start, tokens)]; requests
    that start later than 0 get their earlier tokens from the caller through an earlier step."""
    from xinfer_b200.cache import CacheGroup, CacheManager
    from xinfer_b200.engine.runner import StepAssembler
    cm = CacheManager([CacheGroup(page, pages, window)], max_requests=8)
    asm = StepAssembler(cm, vocab_size=vocab, max_model_len=4096, dtype=dtype, device=DEV)
    return cm, asm


def tolerance(dtype):
    return 3e-5 if dtype == torch.float32 else 2.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from xinfer_b200.config.plan import NormSpec
    from xinfer_b200.parts import build_part
    from xinfer_b200.engine.runner import StepInput
    dim, T = 72, 9
    w = torch.randn(dim) * 0.1 + 1
    part = build_part("norm", NormSpec(kind="rmsnorm", dim=dim, eps=2e-5), "n.", dtype, DEV)
    assert [s.name for s in type(part).weight_specs(part.spec, "n.")] == ["n.weight"]
    part.load(FakeStore({"n.weight": w}))
    assert part.weight.dtype == torch.float32
    cm, asm = context(None, dtype)
    ctx = asm.prepare([StepInput(cm.open_request(), list(range(T)))])
    x = torch.randn(T, dim).to(dtype)
    out = torch.empty(T, dim, dtype=dtype, device=DEV)
    part.forward(out, x.to(DEV), ctx)
    assert (out.float().cpu() - plain.rms_norm(x.float(), w, 2e-5)).abs().max() <= tolerance(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from xinfer_b200.config.plan import FeedForwardSpec
    from xinfer_b200.parts import build_part
    from xinfer_b200.engine.runner import StepInput
    H, I, T = 40, 104, 11
    w = {"f.gate_proj.weight": torch.randn(I, H) * 0.3, "f.up_proj.weight": torch.randn(I, H) * 0.3,
         "f.down_proj.weight": torch.randn(H, I) * 0.3}
    w = {k: v.to(dtype) for k, v in w.items()}
    part = build_part("feed_forward", FeedForwardSpec(kind="swiglu", hidden=H, intermediate=I), "f.", dtype, DEV)
    assert sorted(s.name for s in type(part).weight_specs(part.spec, "f.")) == sorted(w)
    part.load(FakeStore(w))
    cm, asm = context(None, dtype)
    ctx = asm.prepare([StepInput(cm.open_request(), list(range(T)))])
    x = torch.randn(T, H).to(dtype)
    out = part.forward(x.to(DEV), ctx)
    ref = plain.mlp_block(x.float(), {k: v.float() for k, v in w.items()}, "f.")
    assert (out.float().cpu() - ref).abs().max() <= tolerance(dtype) * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,window,page", [(6, 2, 16, None, 8), (4, 4, 48, 13, 4), (8, 1, 64, None, 16)])
def test_attention_part_in_portions(dtype, nh, nkv, d, window, page):
    """The mixer alone: a sequence fed in three portions through the paged cache equals the plain
    attention block on the whole sequence."""
    from xinfer_b200.config.plan import AttentionSpec, RopeSpec
    from xinfer_b200.parts import LayerCache, build_part
    from xinfer_b200.engine.runner import StepInput
    H, T, eps, theta = 56, 45, 1e-5, 30000.0
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=d, hidden_size=H, rms_norm_eps=eps,
               rope_theta=theta, sliding_window=window)
    w = {"a.q_proj.weight": torch.randn(nh * d, H) * 0.2, "a.k_proj.weight": torch.randn(nkv * d, H) * 0.2,
         "a.v_proj.weight": torch.randn(nkv * d, H) * 0.2, "a.o_proj.weight": torch.randn(H, nh * d) * 0.2,
         "a.q_norm.weight": torch.randn(d) * 0.1 + 1.5, "a.k_norm.weight": torch.randn(d) * 0.1 + 1.5}
    w = {k: v.to(dtype) for k, v in w.items()}
    spec = AttentionSpec(kind="attention", hidden=H, num_heads=nh, num_kv_heads=nkv, head_dim=d, scale=d ** -0.5,
                         qk_norm=True, qk_norm_eps=eps, window=window,
                         rope=RopeSpec(kind="rope", head_dim=d, rotary_dim=d, theta=theta, max_positions=128))
    part = build_part("mixer", spec, "a.", dtype, DEV)
    part.load(FakeStore(w))
    need = part.cache_need()
    assert [n for n, _ in need.tensors] == ["k", "v"] and need.window == window and need.page_size is None
    assert all(t.shape == (nkv, d) and t.page_shape(40, page) == (40, nkv, page, d) for _, t in need.tensors)
    cm, asm = context(None, dtype, page=page, pages=40, window=window)
    cache = LayerCache.of_keys_and_values(torch.zeros(40, nkv, page, d, dtype=dtype, device=DEV), torch.zeros(40, nkv, page, d, dtype=dtype, device=DEV), 0, page)
    x = (torch.randn(T, H)).to(dtype)
    slot = cm.open_request()
    outs, at = [], 0
    for n in (17, 2, 26):
        entry = StepInput(slot, list(range(n)))
        ctx = asm.prepare([entry])
        outs.append(part.forward(x[at:at + n].to(DEV).contiguous(), ctx, cache, None, True).clone())
        cm.advance(slot, at + n)
        at += n
    got = torch.cat(outs).float().cpu()
    ref = plain.attention_block(x.float(), {k: v.float() for k, v in w.items()}, "a.", cfg, list(range(T)))
    assert int(asm.err) == 0
    assert (got - ref).abs().max() <= tolerance(dtype) * max(1.0, ref.abs().max().item()), (got - ref).abs().max()


def test_position_part_tables():
    from xinfer_b200.config.plan import RopeSpec
    from xinfer_b200.parts import build_part
    part = build_part("position", RopeSpec(kind="rope", head_dim=64, rotary_dim=32, theta=5e5, max_positions=300, layout="interleaved"), "", torch.bfloat16, DEV)
    t = part.rotary()
    assert t.cos.dtype == torch.float32 and t.cos.shape == (300, 16) and t.rotary_dim == 32 and t.interleaved
    ang = plain.rope_angles(range(300), 32, 5e5)
    assert (t.cos.cpu() - torch.cos(ang.double()).float()).abs().max() < 2e-6
    assert (t.sin.cpu() - torch.sin(ang.double()).float()).abs().max() < 2e-6
    with pytest.raises(ValueError):
        build_part("position", RopeSpec(kind="rope", head_dim=16, rotary_dim=18, theta=1e4, max_positions=8), "", torch.float32, DEV)
    with pytest.raises(ValueError):
        build_part("position", RopeSpec(kind="nonesuch"), "", torch.float32, DEV)


def test_layer_order_is_data(model_folders, tmp_path):
    """The run list [0, 1, 1, 0 reading run 0's cache] over the two blocks of tiny A: whole prompt
    and token-by-token agree, and both equal a plain restatement of that order."""
    from xinfer_b200.config import Qwen3Config
    from xinfer_b200.config.plan import LayerRun
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.models import DecoderModel
    from xinfer_b200.weights import WeightStore
    from helpers import TINY, prompts_for
    folder = model_folders("A", torch.float32)
    cfg, w = plain.load_folder(folder)
    plan = Qwen3Config.from_dict(TINY["A"][0]).plan()
    plan = dataclasses.replace(plan, runs=(LayerRun(0), LayerRun(1), LayerRun(1), LayerRun(0, cache_from=0)))
    model = DecoderModel(plan, torch.float32, DEV)
    model.load(WeightStore(folder))
    r = ModelRunner(folder, "float32", block_size=16, num_blocks=16, max_num_seqs=2, model=model)
    assert [c is not None for c in r.layer_caches] == [True, True, True, False]
    ids = prompts_for("A", [40])[0]
    s = r.open_request()
    whole = r.step([StepInput(s, ids, range(40))]).cpu().clone()
    r.close_request(s)
    s = r.open_request()
    parts = [r.step([StepInput(s, ids[:9], range(9))]).cpu().clone()]
    for i in range(9, 40):
        parts.append(r.step([StepInput(s, ids[i:i + 1], [0])]).cpu().clone())
    r.check_errors()
    assert torch.equal(torch.cat(parts), whole)

    # plain restatement: run 3 uses block 0's weights but the keys/values that run 0 produced
    x = plain.embed(ids, w["model.embed_tokens.weight"])
    pos = list(range(40))
    kv0 = {}

    def layer(x, i, reuse=None):
        p = f"model.layers.{i}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        a = p + "self_attn."
        nh, nkv, d = 4, 2, 16
        q = plain.rms_norm(plain.linear(h, w[a + "q_proj.weight"]).view(40, nh, d), w[a + "q_norm.weight"], cfg["rms_norm_eps"])
        ang = plain.rope_angles(pos, d, cfg["rope_theta"])
        q = plain.apply_rope(q, ang)
        if reuse is None:
            k = plain.apply_rope(plain.rms_norm(plain.linear(h, w[a + "k_proj.weight"]).view(40, nkv, d), w[a + "k_norm.weight"], cfg["rms_norm_eps"]), ang)
            v = plain.linear(h, w[a + "v_proj.weight"]).view(40, nkv, d)
        else:
            k, v = reuse
        o = plain.causal_attention(q, k, v, d ** -0.5)
        r1 = x + plain.linear(o.reshape(40, nh * d), w[a + "o_proj.weight"])
        h2 = plain.rms_norm(r1, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        return r1 + plain.mlp_block(h2, w, p + "mlp."), (k, v)
    x, kv = layer(x, 0)
    x, _ = layer(x, 1)
    x, _ = layer(x, 1)
    x, _ = layer(x, 0, reuse=kv)
    ref = plain.linear(plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])
    assert (whole - ref).abs().max() < 2e-5


def test_a_step_reads_token_ids_that_a_sampler_left_on_the_device(model_folders):
    """A token id -1 - i stands for sampled_tokens[i]: the step's logits equal those of the same
    step with the ids given by the host; an id beyond the buffer is reported, not followed."""
    from xinfer_b200.engine.runner import ModelRunner, StepError, StepInput
    folder = model_folders("A", torch.float32)
    r = ModelRunner(folder, "float32", block_size=16, num_blocks=16, max_num_seqs=3)
    a, b = r.open_request(), r.open_request()
    r.step([StepInput(a, [5, 6, 7], []), StepInput(b, [9], [])])
    r.sampled_tokens[:3] = torch.tensor([41, 250, 17], dtype=torch.int32)
    got = r.step([StepInput(a, [r.ahead_token(2)], [0]), StepInput(b, [r.ahead_token(0)], [0])]).cpu().clone()
    r.check_errors()
    c, d = r.open_request(), None
    r.close_request(a); r.close_request(b)
    a, b = r.open_request(), r.open_request()
    r.step([StepInput(a, [5, 6, 7], []), StepInput(b, [9], [])])
    want = r.step([StepInput(a, [17], [0]), StepInput(b, [41], [0])]).cpu().clone()
    assert torch.equal(got, want)
    with pytest.raises(StepError, match="token ids"):
        r.step([StepInput(a, [-5], [0])])                  # beyond the three ids the buffer holds
    r.sampled_tokens[0] = 100000                            # what the device finds there is checked too
    r.step([StepInput(a, [r.ahead_token(0)], [0])])
    with pytest.raises(StepError, match="token id"):
        r.check_errors()
