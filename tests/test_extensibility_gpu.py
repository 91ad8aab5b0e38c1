"""Parts and an architecture registered from outside the package, with no change to it.

A toy mixer with fixed-size state of its own (a running mean of its inputs), a toy
architecture whose layers differ from one another (attention in one, the toy mixer in
another, feed-forwards of different widths), and an execution order that runs a layer twice
and lets a run read the keys and values another run stored.  Everything is defined here,
registered through the public registry, built from a model folder written by the
random-weights mode, and stepped under the same cuts as the real model.  None of it is a
model of anyone's.
"""

import dataclasses

import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def define_toy():
    from enginekernel_b200 import registry
    from enginekernel_b200.config.base import ModelConfig, key
    from enginekernel_b200.parts.base import Mixer
    from enginekernel_b200.parts.spec import (CacheSpec, LayerSpec, ModelSpec, PartSpec, RunSpec,
                                              TensorSpec)

    class RunningMean(Mixer):
        """y_t = W . mean(x_0..x_t) per sequence; state: the sum so far and the count."""

        @classmethod
        def tensors(cls, spec):
            h = spec.params["hidden_size"]
            return [TensorSpec(spec.weights["w"], (h, h))]

        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.hidden = int(self.param("hidden_size"))

        def cache_spec(self):
            return CacheSpec("state", shape=(self.hidden + 1,))

        def load(self, tensors):
            self.w = tensors[self.spec.weights["w"]].float()

        def forward(self, x, ctx, entry, writes_cache=True):
            out = torch.empty(ctx.n_tokens, self.hidden, dtype=torch.float32, device=x.device)
            cu = ctx.host_cu_seqlens
            for b in range(ctx.n_seqs):
                lo, hi = cu[b], cu[b + 1]
                state = entry.state[ctx.host_token_slot[lo]]
                xs = x[lo:hi].float()
                sums = state[:self.hidden] + torch.cumsum(xs, 0)
                counts = state[self.hidden] + torch.arange(1, hi - lo + 1, device=x.device)
                out[lo:hi] = (sums / counts[:, None]) @ self.w.t()
                if writes_cache:
                    state[:self.hidden] = sums[-1]
                    state[self.hidden] = counts[-1]
            return out.to(self.dtype)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "ToyMixedForCausalLM"
        hidden_size: int = key("hidden_size")
        vocab_size: int = key("vocab_size")
        heads: int = key("heads")
        kv_heads: int = key("kv_heads")
        head_dim: int = key("head_dim")
        widths: int = key("ff_width")
        eps: float = key("eps")
        theta: float = key("theta")
        max_positions: int = key("max_positions")

    def build(cfg):
        h = cfg.hidden_size

        def norms(p):
            return {n: PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": f"{p}.{n}.gain"})
                    for n in ("pre_mixer", "pre_feed_forward")}

        def ff(p, width):
            return PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": width},
                            {"gate": f"{p}.ff.gate", "up": f"{p}.ff.up", "down": f"{p}.ff.down"})

        def attn(p):
            return PartSpec("attention", {
                "hidden_size": h, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                "head_dim": cfg.head_dim, "scale": cfg.head_dim ** -0.5, "qk_norm_eps": cfg.eps,
                "window": None,
                "position": PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.theta,
                                                   "rotary_dim": cfg.head_dim})},
                {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "o": f"{p}.o",
                 "q_norm": f"{p}.qn", "k_norm": f"{p}.kn"})

        layers = [
            LayerSpec(PartSpec("pre_norm"), attn("l0"), ff("l0", cfg.widths), norms("l0")),
            LayerSpec(PartSpec("pre_norm"), PartSpec("running_mean", {"hidden_size": h}, {"w": "l1.w"}),
                      ff("l1", cfg.widths + 16), norms("l1")),
            LayerSpec(PartSpec("pre_norm"), attn("l2"), ff("l2", cfg.widths), norms("l2")),
        ]
        # layer 0 runs twice (own cache entries 0 and 2); the last run reads entry 0's keys and
        # values with layer 2's queries and stores nothing
        schedule = [RunSpec(0, 0), RunSpec(1, 1), RunSpec(0, 2), RunSpec(2, 0, writes_cache=False)]
        return ModelSpec(
            hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
            embedding=TensorSpec("embed", (cfg.vocab_size, h), "embedding"), layers=layers,
            schedule=schedule, final_norm=PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": "final.gain"}),
            lm_head=TensorSpec("head", (cfg.vocab_size, h)))

    registry.register_part("mixer", "running_mean", RunningMean, replace=True)
    registry.register_architecture("ToyMixedForCausalLM", ToyConfig, build, replace=True)
    return ToyConfig


RAW = {"architectures": ["ToyMixedForCausalLM"], "hidden_size": 64, "vocab_size": 97, "heads": 4,
       "kv_heads": 2, "head_dim": 32, "ff_width": 80, "eps": 1e-5, "theta": 10000.0, "max_positions": 512}


def plain_logits(folder, ids):
    """The toy model on one whole sequence with the plain per-part functions."""
    import json
    import os
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    w = plain.read_weights(folder, torch.float32)
    s, nh, nkv, d, eps = len(ids), c["heads"], c["kv_heads"], c["head_dim"], c["eps"]
    cos, sin = plain.rope_tables(s, d, c["theta"], torch.float32)
    r = w["embed"][torch.tensor(ids)]
    stored = {}

    def ffn(p, m):
        g, u = m @ w[f"{p}.ff.gate"].t(), m @ w[f"{p}.ff.up"].t()
        return (torch.nn.functional.silu(g) * u) @ w[f"{p}.ff.down"].t()

    for p, kind, entry, writes in (("l0", "attn", 0, True), ("l1", "mean", 1, True),
                                   ("l0", "attn", 2, True), ("l2", "attn", 0, False)):
        a = plain.rms_norm(r, w[f"{p}.pre_mixer.gain"], eps)
        if kind == "mean":
            o = (torch.cumsum(a, 0) / torch.arange(1, s + 1)[:, None]) @ w["l1.w"].t()
        else:
            q = plain.qk_norm_rope((a @ w[f"{p}.q"].t()).view(s, nh, d), w[f"{p}.qn"], cos, sin, eps)
            if writes:
                k = plain.qk_norm_rope((a @ w[f"{p}.k"].t()).view(s, nkv, d), w[f"{p}.kn"], cos, sin, eps)
                stored[entry] = (k, (a @ w[f"{p}.v"].t()).view(s, nkv, d))
            k, v = stored[entry]
            o = plain.causal_gqa_attention(q, k, v, d ** -0.5) @ w[f"{p}.o"].t()
        r = r + o
        r = r + ffn(p, plain.rms_norm(r, w[f"{p}.pre_feed_forward.gain"], eps))
    return plain.rms_norm(r, w["final.gain"], eps) @ w["head"].t()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer(tmp_path, dtype):
    from enginekernel_b200 import Engine, registry
    from enginekernel_b200.weights import write_random_model
    ToyConfig = define_toy()
    try:
        cfg = ToyConfig.from_dict(RAW)
        folder = write_random_model(str(tmp_path / "toy"), cfg, seed=4)
        eng = Engine(folder, dtype, max_tokens=2048, max_batch=4)
        kinds = sorted(g.spec.kind for g in eng.cache.groups)
        assert kinds == ["kv", "state"]                      # two groups with storage of their own
        assert eng.cache.entry(1).state.shape[-1] == 65
        g = torch.Generator().manual_seed(0)
        seqs = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (90, 7, 40)]
        wants = [plain_logits(folder, s) for s in seqs]
        tol = helpers.TOL[dtype]
        for s, w in zip(seqs, wants):
            assert helpers.rel_err(helpers.whole(eng, s), w) <= tol
            assert helpers.rel_err(helpers.tail_one_by_one(eng, s, 32), w) <= tol
        # unequal batches twice in a row: slots are used again, so stale state would show
        for _ in range(2):
            got = helpers.batch_then_steps(eng, seqs, [50, 7, 1])
            for gl, w in zip(got, wants):
                assert helpers.rel_err(gl, w) <= tol
    finally:
        registry.unregister_part("mixer", "running_mean")
        registry.unregister_architecture("ToyMixedForCausalLM")


def test_unknown_kinds_are_named():
    from enginekernel_b200 import registry
    with pytest.raises(registry.RegistryError, match="attention"):
        registry.lookup_part("mixer", "no_such_mixer")
