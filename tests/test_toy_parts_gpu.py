"""Toy parts defined here and registered from outside the framework: a feed-forward with routing
(router logits in float32, one expert per token), a position encoding that is no rotation, and a
norm with a bias, put together with the framework's attention into a model whose layers differ and
whose order of layers names one layer twice.  None of them is anyone's model; they show that the
interfaces of the parts carry more than the one architecture that is built."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

HEADS, KV_HEADS, HEAD_DIM = 3, 1, 32
EXPERTS = 5


def register_toys():
    from xinfer_b200.config import register_architecture
    from xinfer_b200.config.plan import (AttentionSpec, pre_norm_block, FeedForwardSpec, LayerRun, ModelPlan, NormSpec,
                                         PartSpec)
    from xinfer_b200.parts import (FeedForward, Norm, PositionEncoding, register_feed_forward, register_norm,
                                   register_position_encoding)
    from xinfer_b200.parts.linear import linear
    from xinfer_b200.weights import WeightSpec

    @dataclass(frozen=True)
    class RoutedSpec(PartSpec):
        hidden: int = 0
        inner: int = 0
        experts: int = 0

    class Routed(FeedForward):
        """p = softmax_float32(x . Wr^T); e = argmax p; out = p_e * W2_e . relu(W1_e . x)."""
        kind = "toy_routed"

        @classmethod
        def weight_specs(cls, spec, prefix):
            out = [WeightSpec(prefix + "router.weight", (spec.experts, spec.hidden))]
            for e in range(spec.experts):
                out += [WeightSpec(prefix + f"experts.{e}.w1.weight", (spec.inner, spec.hidden)),
                        WeightSpec(prefix + f"experts.{e}.w2.weight", (spec.hidden, spec.inner))]
            return out

        def load(self, store):
            s, p = self.spec, self.prefix
            self.router = store.get(p + "router.weight", self.device, torch.float32).float()
            self.w1 = [store.get(p + f"experts.{e}.w1.weight", self.device, self.dtype) for e in range(s.experts)]
            self.w2 = [store.get(p + f"experts.{e}.w2.weight", self.device, self.dtype) for e in range(s.experts)]

        def forward(self, x, ctx):
            s = self.spec
            T = x.shape[0]
            ws = ctx.workspace
            logits = ws.get("toy.router", (T, s.experts), torch.float32)
            linear(logits, x.float() if x.dtype != torch.float32 else x, self.router, ctx.err)
            prob = torch.softmax(logits, dim=-1)
            top_p, top_e = prob.max(dim=-1)
            out = ws.get("toy.routed_out", (T, s.hidden), self.dtype)
            out.zero_()
            hid = ws.get("toy.hid", (T, s.inner), self.dtype)
            one = ws.get("toy.one", (T, s.hidden), self.dtype)
            for e in range(s.experts):          # every expert runs on all rows; the mask picks its own
                linear(hid, x, self.w1[e], ctx.err)
                hid.relu_()
                linear(one, hid, self.w2[e], ctx.err)
                mask = (top_e == e)[:, None]
                out += torch.where(mask, (one.float() * top_p[:, None]).to(self.dtype), torch.zeros_like(one))
            return out

    @dataclass(frozen=True)
    class WaveSpec(PartSpec):
        head_dim: int = 0
        rate: float = 0.0

    class Wave(PositionEncoding):
        """q and k are scaled elementwise by 1 + 0.5 cos(rate * position + j): position enters the
        scores without any rotation, through ``apply`` instead of rotary tables."""
        kind = "toy_wave"

        def apply(self, q, k, ctx):
            s = self.spec
            j = torch.arange(s.head_dim, device=q.device, dtype=torch.float32)
            f = 1.0 + 0.5 * torch.cos(ctx.positions.float()[:, None] * s.rate + j[None, :])   # [T, d]
            q.copy_((q.float() * f[:, None, :]).to(q.dtype))
            k.copy_((k.float() * f[:, None, :]).to(k.dtype))

    @dataclass(frozen=True)
    class CenteredSpec(PartSpec):
        dim: int = 0
        eps: float = 0.0

    class Centered(Norm):
        """y = (x - mean) * rsqrt(var + eps) * w + b on x (+ branch), statistics in float32."""
        kind = "toy_centered"

        @classmethod
        def weight_specs(cls, spec, prefix):
            return [WeightSpec(prefix + "weight", (spec.dim,), "norm"), WeightSpec(prefix + "bias", (spec.dim,))]

        def load(self, store):
            self.w = store.get(self.prefix + "weight", self.device, torch.float32).float()
            self.b = store.get(self.prefix + "bias", self.device, torch.float32).float()

        def forward(self, out, x, ctx, branch=None, sum_out=None, rows=None):
            if rows is not None:
                x = x[rows.long()]
                branch = branch[rows.long()] if branch is not None else None
            v = x.float()
            if branch is not None:
                v = (v + branch.float()).to(x.dtype).float()
                if sum_out is not None:
                    sum_out.copy_(v.to(sum_out.dtype))
            mu = v.mean(-1, keepdim=True)
            var = ((v - mu) ** 2).mean(-1, keepdim=True)
            out.copy_(((v - mu) * torch.rsqrt(var + self.spec.eps) * self.w + self.b).to(out.dtype))
            return out

    register_feed_forward("toy_routed", Routed, replace=True)
    register_position_encoding("toy_wave", Wave, replace=True)
    register_norm("toy_centered", Centered, replace=True)

    def plan_of(raw):
        H, V = raw["hidden_size"], raw["vocab_size"]
        blocks = []
        for i, ffn in enumerate(raw["feed_forwards"]):
            mixer = AttentionSpec(kind="attention", hidden=H, num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM,
                                  scale=raw["scale"], qk_norm=False, qk_norm_eps=1e-6,
                                  rope=WaveSpec(kind="toy_wave", head_dim=HEAD_DIM, rate=raw["rate"]))
            if ffn == "routed":
                ff = RoutedSpec(kind="toy_routed", hidden=H, inner=raw["inner"], experts=EXPERTS)
            else:
                ff = FeedForwardSpec(kind="swiglu", hidden=H, intermediate=raw["inner"])
            norm = (CenteredSpec(kind="toy_centered", dim=H, eps=1e-5) if i % 2 else NormSpec(kind="rmsnorm", dim=H, eps=1e-6))
            blocks.append(pre_norm_block(prefix=f"model.layers.{i}.", norm_in=norm, mixer=mixer,
                                    norm_post=NormSpec(kind="rmsnorm", dim=H, eps=1e-6), feed_forward=ff))
        return ModelPlan(architecture="ToyPartsForTest", vocab_size=V, hidden=H, embed_name="model.embed_tokens.weight",
                         blocks=tuple(blocks), runs=tuple(LayerRun(i) for i in raw["order"]),
                         final_norm=NormSpec(kind="rmsnorm", dim=H, eps=1e-6), final_norm_name="model.norm.",
                         head_name=None, max_positions=512)
    register_architecture("ToyPartsForTest", lambda raw: dict(raw), plan_of, replace=True)


def plain_toy(raw, w, ids):
    T, H = len(ids), raw["hidden_size"]
    x = plain.embed(ids, w["model.embed_tokens.weight"])
    pos = torch.arange(T, dtype=torch.float32)
    wave = (1.0 + 0.5 * torch.cos(pos[:, None] * raw["rate"] + torch.arange(HEAD_DIM, dtype=torch.float32)[None, :])).to(x.dtype)
    for i in raw["order"]:
        p = f"model.layers.{i}."
        if i % 2:
            mu = x.mean(-1, keepdim=True)
            var = ((x - mu) ** 2).mean(-1, keepdim=True)
            h = (x - mu) * torch.rsqrt(var + 1e-5) * w[p + "input_layernorm.weight"] + w[p + "input_layernorm.bias"]
        else:
            h = plain.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
        a = p + "self_attn."
        q = plain.linear(h, w[a + "q_proj.weight"]).view(T, HEADS, HEAD_DIM) * wave[:, None, :]
        k = plain.linear(h, w[a + "k_proj.weight"]).view(T, KV_HEADS, HEAD_DIM) * wave[:, None, :]
        v = plain.linear(h, w[a + "v_proj.weight"]).view(T, KV_HEADS, HEAD_DIM)
        o = plain.causal_attention(q, k, v, raw["scale"])
        r1 = x + plain.linear(o.reshape(T, HEADS * HEAD_DIM), w[a + "o_proj.weight"])
        h2 = plain.rms_norm(r1, w[p + "post_attention_layernorm.weight"], 1e-6)
        if raw["feed_forwards"][i] == "routed":
            prob = torch.softmax(plain.linear(h2, w[p + "mlp.router.weight"]), dim=-1)
            top_p, top_e = prob.max(-1)
            f = torch.zeros(T, H, dtype=x.dtype)
            for t in range(T):
                e = int(top_e[t])
                hid = torch.relu(plain.linear(h2[t:t + 1], w[p + f"mlp.experts.{e}.w1.weight"]))
                f[t] = top_p[t] * plain.linear(hid, w[p + f"mlp.experts.{e}.w2.weight"])[0]
        else:
            f = plain.mlp_block(h2, w, p + "mlp.")
        x = r1 + f
    return plain.linear(plain.rms_norm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"])


def test_toy_feed_forward_position_encoding_and_norm_are_registered_and_stepped(tmp_path):
    from xinfer_b200.config import unregister_architecture
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts import unregister
    from xinfer_b200.weights import write_random_model
    register_toys()
    try:
        raw = dict(architectures=["ToyPartsForTest"], vocab_size=113, hidden_size=72, inner=88, scale=0.2, rate=0.37,
                   feed_forwards=["routed", "swiglu", "routed"], order=[0, 1, 2, 1])

        def widen(name, t):     # routing and attention must not be flat
            if name.endswith("router.weight"):
                return t.float() * 40.0
            if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
                return t.float() * 4.0
            return None
        folder = write_random_model(str(tmp_path / "toy"), raw, seed=9, dtype=torch.float32, std=0.08, override=widen)
        _, w = plain.load_folder(folder)
        r = ModelRunner(folder, "float32", block_size=8, num_blocks=48, max_num_seqs=3)
        assert len(r.layer_caches) == 4 and all(c is not None for c in r.layer_caches), "a layer run twice has two caches"
        rng = np.random.default_rng(3)
        a, b = rng.integers(0, 113, 61).tolist(), rng.integers(0, 113, 40).tolist()
        ref_a, ref_b = plain_toy(raw, w, a), plain_toy(raw, w, b)
        # float32 rounding of the plain implementation itself, measured against float64: the bound
        # for the engine's float32 is a small multiple of it
        _, w64 = plain.load_folder(folder, dtype=torch.float64)
        own = max(float((plain_toy(raw, w64, p).float() - r).abs().max()) for p, r in ((a, ref_a), (b, ref_b)))
        tol = max(3e-5, 4.0 * own)
        # the router must really spread the tokens, or the test shows nothing
        h_probe = plain.linear(plain.embed(a, w["model.embed_tokens.weight"]), w["model.layers.0.mlp.router.weight"])
        assert len(set(h_probe.argmax(-1).tolist())) >= 3
        sa = r.open_request()
        whole = r.step([StepInput(sa, a, range(len(a)))]).cpu().clone()
        assert (whole - ref_a).abs().max() < tol
        r.close_request(sa)
        sa, sb = r.open_request(), r.open_request()
        got_a, got_b = [], []
        got_a.append(r.step([StepInput(sa, a[:23], range(23))]).cpu().clone())
        out = r.step([StepInput(sb, b[:37], range(37)), StepInput(sa, a[23:25], range(2))]).cpu().clone()
        got_b.append(out[:37]); got_a.append(out[37:])
        out = r.step([StepInput(sa, a[25:], range(len(a) - 25)), StepInput(sb, b[37:38], [0])]).cpu().clone()
        got_a.append(out[:len(a) - 25]); got_b.append(out[len(a) - 25:])
        for j in range(38, len(b)):
            got_b.append(r.step([StepInput(sb, b[j:j + 1], [0])]).cpu().clone())
        r.check_errors()
        assert (torch.cat(got_a) - ref_a).abs().max() < tol
        assert (torch.cat(got_b) - ref_b).abs().max() < tol
    finally:
        unregister_architecture("ToyPartsForTest")
        unregister("feed_forward", "toy_routed")
        unregister("position", "toy_wave")
        unregister("norm", "toy_centered")
