"""Arrangements and caches other than the built architecture's, made of toy parts that are
defined and registered here, with no change to the framework's files:

* blocks whose programs differ from the pre-norm block: a sandwich block with four norms, a
  parallel block (mixer and feed-forward read the same norm), a post-norm block (norm of the sum,
  in place of the stream), a block without a feed-forward;
* a mixer that caches ONE latent tensor per token (not keys and values), in pages of its own size,
  beside attention layers whose pages have another size (two cache groups);
* a plan with an embedding scale, a logit scale and a logit soft cap.

The model is replayed whole, with the last 32 tokens one by one, in portions of changing size and
mixed with other requests over a pool so small that pages are used again, and compared at every
position with a plain restatement written below.  None of this is anyone's model."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import build_all_modes, replay_in_process

pytestmark = pytest.mark.gpu

H, V, LATENT, INNER = 80, 131, 24, 112
HEADS, KV_HEADS, HEAD_DIM = 4, 2, 16
EMBED_SCALE, LOGIT_SCALE, SOFTCAP = 3.0, 2.0, 4.0
LATENT_PAGE = 4
ARCH = "ToyArrangementsForTest"
EPS = 1e-6


def register_toys():
    from xinfer_b200.config import register_architecture
    from xinfer_b200.config.plan import (AttentionSpec, BlockOp, BlockSpec, FeedForwardSpec, LayerRun, ModelPlan,
                                         NormSpec, PartSpec, RopeSpec)
    from xinfer_b200.parts import CacheTensor, Mixer, PagedCacheNeed, register_mixer
    from xinfer_b200.parts.linear import linear
    from xinfer_b200.weights import WeightSpec

    @dataclass(frozen=True)
    class LatentSpec(PartSpec):
        hidden: int = 0
        latent: int = 0
        page_size: int = 4

    class LatentMean(Mixer):
        """c[t] = Wc . x[t] is cached, one vector per token; out[t] = Wo . mean(c[0..t])."""
        kind = "toy_latent"

        @classmethod
        def weight_specs(cls, spec, prefix):
            return [WeightSpec(prefix + "down.weight", (spec.latent, spec.hidden)),
                    WeightSpec(prefix + "up.weight", (spec.hidden, spec.latent))]

        def load(self, store):
            self.wc = store.get(self.prefix + "down.weight", self.device, self.dtype, operand=True)
            self.wo = store.get(self.prefix + "up.weight", self.device, self.dtype, operand=True)

        def cache_need(self):
            # one tensor per token, [page, slot, latent], in float32 whatever the engine's dtype is
            return PagedCacheNeed((("latent", CacheTensor((self.spec.latent,), torch.float32, 0)),), None, self.spec.page_size)

        def forward(self, x, ctx, cache, state, writes_cache=True):
            T = x.shape[0]
            L, ps = self.spec.latent, cache.page_size
            pages = cache["latent"]
            assert tuple(pages.shape[1:]) == (ps, L) and pages.dtype == torch.float32
            c = ctx.workspace.get("toy.latent", (T, L), self.dtype)
            linear(c, x, self.wc, ctx.err)
            table = ctx.tables[cache.group].view(ctx.num_entries, ctx.strides[cache.group])
            means = ctx.workspace.get("toy.latent_mean", (T, L), self.dtype)
            means.zero_()
            for b in range(ctx.real_entries):
                lo, hi = int(ctx.h_q_start[b]), int(ctx.h_q_start[b + 1])
                start = int(ctx.h_start_pos[b])
                pos = torch.arange(start, start + hi - lo, device=x.device)
                if writes_cache:        # write this step's latents to their pages before reading
                    pages[table[b, pos // ps].long(), pos % ps] = c[lo:hi].float()
                allpos = torch.arange(0, start + hi - lo, device=x.device)
                seen = pages[table[b, allpos // ps].long(), allpos % ps]            # [start + n, L], through the block table
                run = torch.cumsum(seen, 0)[start:] / (pos + 1).float()[:, None]
                means[lo:hi] = run.to(self.dtype)
            out = ctx.workspace.get("toy.latent_out", (T, self.spec.hidden), self.dtype)
            return linear(out, means, self.wo, ctx.err)

    register_mixer("toy_latent", LatentMean, replace=True)

    def plan_of(raw):
        norm = lambda: NormSpec(kind="rmsnorm", dim=H, eps=EPS)
        blocks = []
        for i, (arrangement, mixer_kind) in enumerate(raw["layers"]):
            if mixer_kind == "attention":
                mixer = AttentionSpec(kind="attention", hidden=H, num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM,
                                      scale=HEAD_DIM ** -0.5, qk_norm=True, qk_norm_eps=EPS,
                                      rope=RopeSpec(kind="rope", head_dim=HEAD_DIM, rotary_dim=HEAD_DIM, theta=1e4, max_positions=512))
            else:
                mixer = LatentSpec(kind="toy_latent", hidden=H, latent=LATENT, page_size=LATENT_PAGE)
            ffn = FeedForwardSpec(kind="swiglu", hidden=H, intermediate=INNER)
            if arrangement == "sandwich":        # four norms: before and after each part
                prog = (BlockOp("norm", "x", "h", norm(), "n1."), BlockOp("mixer", "h", "a", mixer, "mix."),
                        BlockOp("norm", "a", "a2", norm(), "n2."), BlockOp("add", "a2", "x"),
                        BlockOp("norm", "x", "h", norm(), "n3."), BlockOp("feed_forward", "h", "f", ffn, "ffn."),
                        BlockOp("norm", "f", "f2", norm(), "n4."), BlockOp("add", "f2", "x"))
            elif arrangement == "parallel":      # both parts read one norm; both branches are added
                prog = (BlockOp("norm", "x", "h", norm(), "n1."), BlockOp("mixer", "h", "a", mixer, "mix."),
                        BlockOp("feed_forward", "h", "f", ffn, "ffn."), BlockOp("add", "a", "x"), BlockOp("add", "f", "x"))
            elif arrangement == "postnorm":      # the stream itself is normed after each sum
                prog = (BlockOp("mixer", "x", "a", mixer, "mix."), BlockOp("add", "a", "x"), BlockOp("norm", "x", "x", norm(), "n1."),
                        BlockOp("feed_forward", "x", "f", ffn, "ffn."), BlockOp("add", "f", "x"), BlockOp("norm", "x", "x", norm(), "n2."))
            else:                                # "mixer_only": no feed-forward at all
                prog = (BlockOp("norm", "x", "h", norm(), "n1."), BlockOp("mixer", "h", "a", mixer, "mix."), BlockOp("add", "a", "x"))
            blocks.append(BlockSpec(f"model.layers.{i}.", prog))
        return ModelPlan(architecture=ARCH, vocab_size=V, hidden=H, embed_name="model.embed_tokens.weight",
                         blocks=tuple(blocks), runs=tuple(LayerRun(i) for i in range(len(blocks))),
                         final_norm=norm(), final_norm_name="model.norm.", head_name="lm_head.weight", max_positions=512,
                         embed_scale=EMBED_SCALE, logit_scale=LOGIT_SCALE, logit_softcap=SOFTCAP)

    register_architecture(ARCH, lambda raw: dict(raw), plan_of, replace=True)


# ---------------------------------------------------------------------------------------------
# the plain restatement: whole sequences, no cache
# ---------------------------------------------------------------------------------------------
def plain_toy(raw, w, ids, round_to=None):
    """``round_to`` = torch.bfloat16 rounds activations where a bfloat16 engine stores them."""
    rnd = lambda t: plain._round(t, round_to)
    T = len(ids)
    cfg = dict(num_attention_heads=HEADS, num_key_value_heads=KV_HEADS, head_dim=HEAD_DIM, hidden_size=H,
               rms_norm_eps=EPS, rope_theta=1e4)
    norm = lambda t, name: rnd(plain.rms_norm(t, w[name + "weight"], EPS))
    x = rnd(plain.embed(ids, w["model.embed_tokens.weight"]) * EMBED_SCALE)
    for i, (arrangement, mixer_kind) in enumerate(raw["layers"]):
        p = f"model.layers.{i}."

        def mixer(h):
            if mixer_kind == "attention":
                return plain.attention_block(h, w, p + "mix.", cfg, list(range(T)), round_to)
            c = rnd(plain.linear(h, w[p + "mix.down.weight"])).float()          # cached in float32
            means = rnd((torch.cumsum(c, 0) / torch.arange(1, T + 1, dtype=torch.float32)[:, None]).to(h.dtype))
            return rnd(plain.linear(means, w[p + "mix.up.weight"]))

        ffn = lambda h: plain.mlp_block(h, w, p + "ffn.", round_to)
        if arrangement == "sandwich":
            x = rnd(x + norm(mixer(norm(x, p + "n1.")), p + "n2."))
            x = rnd(x + norm(ffn(norm(x, p + "n3.")), p + "n4."))
        elif arrangement == "parallel":
            h = norm(x, p + "n1.")
            a, f = mixer(h), ffn(h)
            x = rnd(rnd(x + a) + f)
        elif arrangement == "postnorm":
            x = norm(rnd(x + mixer(x)), p + "n1.")
            x = norm(rnd(x + ffn(x)), p + "n2.")
        else:
            x = rnd(x + mixer(norm(x, p + "n1.")))
    y = norm(x, "model.norm.")
    logits = plain.linear(y, w["lm_head.weight"]).float() * LOGIT_SCALE
    return SOFTCAP * torch.tanh(logits / SOFTCAP)


LAYERS = [("sandwich", "attention"), ("parallel", "toy_latent"), ("postnorm", "attention"),
          ("mixer_only", "toy_latent"), ("sandwich", "toy_latent"), ("parallel", "attention")]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_arrangements_a_latent_cache_and_scaled_ends_in_every_way_of_cutting(dtype, tmp_path):
    from helpers import sharpen
    from xinfer_b200.config import unregister_architecture
    from xinfer_b200.engine.runner import ModelRunner
    from xinfer_b200.parts import unregister
    from xinfer_b200.weights import write_random_model
    register_toys()
    try:
        raw = dict(architectures=[ARCH], layers=LAYERS)
        store = torch.float32 if dtype == "float32" else torch.bfloat16

        def shape_weights(name, t):      # attention must not be flat; the latent branch must matter
            if name.endswith("mix.up.weight"):
                return t.float() * 3.0
            return sharpen(name, t)
        folder = write_random_model(str(tmp_path / "toy"), raw, seed=21, dtype=store, std=0.08, override=shape_weights)
        _, w = plain.load_folder(folder)
        rng = np.random.default_rng(4)
        prompts = [rng.integers(0, V, size=n).tolist() for n in (70, 45, 130, 33)]
        tb = build_all_modes(prompts, seed=3)
        page = 8
        runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=8)
        # two cache groups: attention's pages of 8 tokens and the latent mixer's pages of 4
        assert sorted(g.page_size for g in runner.cache.groups) == [LATENT_PAGE, page]
        latent = [c for c in runner.layer_caches if "latent" in c.tensors]
        assert len(latent) == 3 and all(set(c.tensors) == {"latent"} and c.page_size == LATENT_PAGE for c in latent)
        assert all(c["latent"].shape == (tb.peak // LATENT_PAGE, LATENT_PAGE, LATENT) for c in latent)
        out = replay_in_process(runner, tb.steps)
        runner.cache.check_consistent()
        assert all(runner.cache.free_pages(g) == grp.num_pages for g, grp in enumerate(runner.cache.groups))

        ref = [plain_toy(raw, w, p).numpy() for p in prompts]
        if dtype == "float32":
            _, w64 = plain.load_folder(folder, dtype=torch.float64)
            own = max(float(np.abs(plain_toy(raw, w64, p).float().numpy() - r).max()) for p, r in zip(prompts, ref))
            tol = [max(2e-5, 4.0 * own)] * len(prompts)
        else:
            tol = [3.0 * np.abs(plain_toy(raw, w, p, round_to=torch.bfloat16).numpy() - r).max() for p, r in zip(prompts, ref)]
        seen = {}
        for step, rows in tb.rows.items():
            got = out[step]
            assert got.shape[0] == len(rows)
            for r, ((mode, i), pos) in enumerate(rows):
                d = float(np.abs(got[r] - ref[i][pos]).max())
                assert d <= tol[i], f"{dtype} {mode}: request {i} position {pos} (step {step}) differs by {d:.3g} > {tol[i]:.3g}"
                seen.setdefault((mode, i), set()).add(pos)
        for mode in ("whole", "tail", "portions", "mixed"):
            for i, p in enumerate(prompts):
                assert seen[(mode, i)] == set(range(len(p))), (mode, i)
        # the soft cap really bit, and the embedding scale really mattered
        assert np.abs(ref[0]).max() <= SOFTCAP and np.abs(ref[0]).max() > 0.5 * SOFTCAP
    finally:
        unregister_architecture(ARCH)
        unregister("mixer", "toy_latent")
