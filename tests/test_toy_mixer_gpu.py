"""A toy mixer with state of its own, defined here, is registered, built and stepped without a
change to the framework's files: a running mean over the request's tokens, kept in the request's
state slot, in a model that alternates it with attention layers."""

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def register_toy():
    from xinfer_b200.config import register_architecture
    from xinfer_b200.config.plan import (AttentionSpec, pre_norm_block, FeedForwardSpec, LayerRun, ModelPlan, NormSpec,
                                         PartSpec, RopeSpec)
    from xinfer_b200.parts import Mixer, register_mixer
    from xinfer_b200.parts.linear import linear
    from xinfer_b200.weights import WeightSpec
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class RunningMeanSpec(PartSpec):
        hidden: int = 0

    class RunningMean(Mixer):
        """out[t] = W . mean(x[0..t]) over the request's tokens so far."""
        kind = "running_mean"

        @classmethod
        def weight_specs(cls, spec, prefix):
            return [WeightSpec(prefix + "mix.weight", (spec.hidden, spec.hidden))]

        def load(self, store):
            self.w = store.get(self.prefix + "mix.weight", self.device, self.dtype)

        def state_need(self):
            return {"sum": ((self.spec.hidden,), torch.float32), "count": ((1,), torch.float32)}

        def forward(self, x, ctx, cache, state, writes_cache=True):
            T, H = x.shape
            means = ctx.workspace.get("toy.means", (T, H), self.dtype)
            means.zero_()
            for b in range(ctx.real_entries):
                lo, hi = int(ctx.h_q_start[b]), int(ctx.h_q_start[b + 1])
                slot = int(ctx.h_slots[b])
                run = state["sum"][slot] + torch.cumsum(x[lo:hi].float(), 0)
                cnt = state["count"][slot] + torch.arange(1, hi - lo + 1, device=x.device, dtype=torch.float32)
                means[lo:hi] = (run / cnt[:, None]).to(self.dtype)
                state["sum"][slot] = run[-1]
                state["count"][slot] = cnt[-1:]
            out = ctx.workspace.get("toy.out", (T, H), self.dtype)
            return linear(out, means, self.w)

    register_mixer("running_mean", RunningMean, replace=True)

    def plan_of(raw):
        H, V = raw["hidden_size"], raw["vocab_size"]
        blocks = []
        for i, kind in enumerate(raw["mixers"]):
            if kind == "attention":
                mixer = AttentionSpec(kind="attention", hidden=H, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                                      qk_norm=True, qk_norm_eps=1e-6,
                                      rope=RopeSpec(kind="rope", head_dim=16, rotary_dim=16, theta=1e4, max_positions=256))
            else:
                mixer = RunningMeanSpec(kind="running_mean", hidden=H)
            blocks.append(pre_norm_block(prefix=f"model.layers.{i}.", norm_in=NormSpec(kind="rmsnorm", dim=H, eps=1e-6), mixer=mixer,
                                    norm_post=NormSpec(kind="rmsnorm", dim=H, eps=1e-6),
                                    feed_forward=FeedForwardSpec(kind="swiglu", hidden=H, intermediate=2 * H)))
        return ModelPlan(architecture="ToyHybridForTest", vocab_size=V, hidden=H, embed_name="model.embed_tokens.weight",
                         blocks=tuple(blocks), runs=tuple(LayerRun(i) for i in range(len(blocks))),
                         final_norm=NormSpec(kind="rmsnorm", dim=H, eps=1e-6), final_norm_name="model.norm.",
                         head_name="lm_head.weight", max_positions=256)
    register_architecture("ToyHybridForTest", lambda raw: dict(raw), plan_of, replace=True)


def plain_toy(raw, w, ids):
    T = len(ids)
    x = plain.embed(ids, w["model.embed_tokens.weight"])
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, hidden_size=raw["hidden_size"],
               rms_norm_eps=1e-6, rope_theta=1e4)
    for i, kind in enumerate(raw["mixers"]):
        p = f"model.layers.{i}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
        if kind == "attention":
            a = plain.attention_block(h, w, p + "self_attn.", cfg, list(range(T)))
        else:
            means = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
            a = plain.linear(means, w[p + "self_attn.mix.weight"])
        r1 = x + a
        x = r1 + plain.mlp_block(plain.rms_norm(r1, w[p + "post_attention_layernorm.weight"], 1e-6), w, p + "mlp.")
    return plain.linear(plain.rms_norm(x, w["model.norm.weight"], 1e-6), w["lm_head.weight"])


def test_toy_state_mixer_is_registered_built_and_stepped(tmp_path):
    from xinfer_b200.config import unregister_architecture
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts import unregister
    from xinfer_b200.weights import write_random_model
    register_toy()
    try:
        raw = dict(architectures=["ToyHybridForTest"], vocab_size=97, hidden_size=64, mixers=["attention", "running_mean", "running_mean", "attention"])
        folder = write_random_model(str(tmp_path / "toy"), raw, seed=5, dtype=torch.float32, std=0.08)
        _, w = plain.load_folder(folder)
        r = ModelRunner(folder, "float32", block_size=8, num_blocks=32, max_num_seqs=3)
        assert [s is not None for s in r.layer_states] == [False, True, True, False]
        assert [c is not None for c in r.layer_caches] == [True, False, False, True]
        rng = np.random.default_rng(0)
        a, b = rng.integers(0, 97, 50).tolist(), rng.integers(0, 97, 33).tolist()
        ref_a, ref_b = plain_toy(raw, w, a), plain_toy(raw, w, b)
        sa = r.open_request()
        whole = r.step([StepInput(sa, a, range(50))]).cpu().clone()
        assert (whole - ref_a).abs().max() < 3e-5
        r.close_request(sa)
        # the slot is reused: its state must start from zero again; portions and a mixed batch
        sa, sb = r.open_request(), r.open_request()
        got_a, got_b = [], []
        got_a.append(r.step([StepInput(sa, a[:20], range(20))]).cpu().clone())
        out = r.step([StepInput(sb, b[:31], range(31)), StepInput(sa, a[20:22], range(2))]).cpu().clone()
        got_b.append(out[:31]); got_a.append(out[31:])
        out = r.step([StepInput(sa, a[22:], range(28)), StepInput(sb, b[31:32], [0])]).cpu().clone()
        got_a.append(out[:28]); got_b.append(out[28:])
        got_b.append(r.step([StepInput(sb, b[32:], [0])]).cpu().clone())
        r.check_errors()
        assert (torch.cat(got_a) - ref_a).abs().max() < 3e-5
        assert (torch.cat(got_b) - ref_b).abs().max() < 3e-5
    finally:
        unregister_architecture("ToyHybridForTest")
        unregister("mixer", "running_mean")


def register_decay():
    """A second toy mixer with state: s <- decay * s + x[t] per request, out[t] = W . s.  For steps of
    single tokens it takes the requests' slots from the device (``ctx.slots``), so such steps can
    be captured in a CUDA graph and replayed; it says so with ``graph_safe``."""
    from xinfer_b200.config import register_architecture
    from xinfer_b200.config.plan import FeedForwardSpec, LayerRun, ModelPlan, NormSpec, PartSpec, pre_norm_block
    from xinfer_b200.parts import Mixer, register_mixer
    from xinfer_b200.parts.linear import linear
    from xinfer_b200.weights import WeightSpec
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class DecaySpec(PartSpec):
        hidden: int = 0
        decay: float = 0.5

    class Decay(Mixer):
        kind = "toy_decay"
        graph_safe = True

        @classmethod
        def weight_specs(cls, spec, prefix):
            return [WeightSpec(prefix + "mix.weight", (spec.hidden, spec.hidden))]

        def load(self, store):
            self.w = store.get(self.prefix + "mix.weight", self.device, self.dtype, operand=True)

        def state_need(self):
            return {"s": ((self.spec.hidden,), torch.float32)}

        def forward(self, x, ctx, cache, state, writes_cache=True):
            T, H = x.shape
            table = state["s"]                                         # [request slots, H]
            d = self.spec.decay
            acc = ctx.workspace.get("toy.decay_s", (T, H), self.dtype)
            if ctx.fixed_shapes or ctx.all_single:
                # one token per entry: everything from device tensors (padding entries have slot -1)
                slots = ctx.slots[:T].long()
                onehot = (slots[:, None] == torch.arange(table.shape[0], device=x.device)[None, :]).float()   # [T, slots]
                new = (onehot @ table) * d + x.float()                  # each row: its request's state, or zeros for padding
                touched = onehot.sum(0) > 0
                table.copy_(torch.where(touched[:, None], onehot.t() @ new, table))
                acc.copy_(new.to(self.dtype))
            else:
                for b in range(ctx.real_entries):
                    lo, hi = int(ctx.h_q_start[b]), int(ctx.h_q_start[b + 1])
                    s = table[int(ctx.h_slots[b])].clone()
                    for t in range(lo, hi):
                        s = s * d + x[t].float()
                        acc[t] = s.to(self.dtype)
                    table[int(ctx.h_slots[b])] = s
            out = ctx.workspace.get("toy.decay_out", (T, H), self.dtype)
            return linear(out, acc, self.w, ctx.err)

    register_mixer("toy_decay", Decay, replace=True)

    def plan_of(raw):
        H, V = raw["hidden_size"], raw["vocab_size"]
        norm = lambda: NormSpec(kind="rmsnorm", dim=H, eps=1e-6)
        blocks = [pre_norm_block(prefix=f"model.layers.{i}.", norm_in=norm(), mixer=DecaySpec(kind="toy_decay", hidden=H, decay=raw["decay"]),
                                 norm_post=norm(), feed_forward=FeedForwardSpec(kind="swiglu", hidden=H, intermediate=2 * H))
                  for i in range(raw["layers"])]
        return ModelPlan(architecture="ToyDecayForTest", vocab_size=V, hidden=H, embed_name="model.embed_tokens.weight",
                         blocks=tuple(blocks), runs=tuple(LayerRun(i) for i in range(len(blocks))),
                         final_norm=norm(), final_norm_name="model.norm.", head_name="lm_head.weight", max_positions=256)
    register_architecture("ToyDecayForTest", lambda raw: dict(raw), plan_of, replace=True)


def plain_decay(raw, w, ids, round_to=None):
    rnd = lambda t: plain._round(t, round_to)
    T = len(ids)
    x = plain.embed(ids, w["model.embed_tokens.weight"])
    for i in range(raw["layers"]):
        p = f"model.layers.{i}."
        h = rnd(plain.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6))
        s, rows = torch.zeros(raw["hidden_size"]), []
        for t in range(T):
            s = s * raw["decay"] + h[t].float()
            rows.append(s)
        a = rnd(plain.linear(rnd(torch.stack(rows).to(h.dtype)), w[p + "self_attn.mix.weight"]))
        r1 = rnd(x + a)
        x = rnd(r1 + plain.mlp_block(rnd(plain.rms_norm(r1, w[p + "post_attention_layernorm.weight"], 1e-6)), w, p + "mlp.", round_to))
    return plain.linear(rnd(plain.rms_norm(x, w["model.norm.weight"], 1e-6)), w["lm_head.weight"])


def test_a_stateful_mixer_that_reads_slots_on_the_device_decodes_from_cuda_graphs(tmp_path):
    """Decode steps of a model whose mixers keep per-request state are replayed from CUDA graphs:
    the state rows are addressed through the step's device metadata, the capture's trial runs leave
    the state as it was, batches shrink and grow across graph buckets."""
    from xinfer_b200.config import unregister_architecture
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts import unregister
    from xinfer_b200.weights import write_random_model
    register_decay()
    try:
        raw = dict(architectures=["ToyDecayForTest"], vocab_size=101, hidden_size=64, layers=2, decay=0.6)
        folder = write_random_model(str(tmp_path / "toy"), raw, seed=8, dtype=torch.bfloat16, std=0.08)
        _, w = plain.load_folder(folder)
        r = ModelRunner(folder, "bfloat16", block_size=8, num_blocks=8, max_num_seqs=3)
        assert r.has_state and r._graph_safe
        rng = np.random.default_rng(1)
        seqs = [rng.integers(0, 101, n).tolist() for n in (40, 31, 22)]
        ref = [plain_decay(raw, w, s) for s in seqs]
        tol = [3.0 * float((plain_decay(raw, w, s, round_to=torch.bfloat16) - f).abs().max()) for s, f in zip(seqs, ref)]
        slots = [r.open_request() for _ in seqs]
        heads = (9, 5, 2)
        got = [[] for _ in seqs]
        out = r.step([StepInput(slots[i], seqs[i][:heads[i]], range(heads[i])) for i in range(3)]).float().cpu()   # prompts, launched
        assert not r.last_used_graph
        at = 0
        for i in range(3):
            got[i].append(out[at:at + heads[i]].clone()); at += heads[i]
        done = list(heads)
        graphs = 0
        while any(done[i] < len(seqs[i]) for i in range(3)):
            live = [i for i in range(3) if done[i] < len(seqs[i])]
            out = r.step([StepInput(slots[i], seqs[i][done[i]:done[i] + 1], [0]) for i in live], allow_graph=True).float().cpu()
            graphs += r.last_used_graph
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1].clone()); done[i] += 1
        r.check_errors()
        assert graphs == len(seqs[0]) - heads[0] and len(r._graphs) >= 2      # buckets of 3, 2 and 1 requests
        for i in range(3):
            d = float((torch.cat(got[i]) - ref[i]).abs().max())
            assert d <= tol[i], (i, d, tol[i])
    finally:
        unregister_architecture("ToyDecayForTest")
        unregister("mixer", "toy_decay")
