"""Parts and an architecture registered from outside the package, with no change to it.

A toy mixer with fixed-size state of its own (a running mean of its inputs), a toy
architecture whose layers differ from one another (attention in one, the toy mixer in
another, feed-forwards of different widths), and an execution order that runs a layer twice
and lets a run read the keys and values another run stored; and a second toy architecture
with a routed feed-forward (one expert a token) and a position encoding of its own inside the
framework's attention.  Everything is defined here, registered through the public registry, built from a model folder written by the
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
            """Device tensors only (no host copy of positions or slots, nothing that waits for the
            device), so the same code runs in steps the host lays out and inside the captured
            decode step of ``generate``.  Rows whose position is negative belong to sequences that
            have ended: they contribute nothing and leave the state alone."""
            t, h = ctx.n_tokens, self.hidden
            dev = x.device
            pos, slots = ctx.positions[:t].long(), ctx.token_slot[:t].long()
            active = pos >= 0
            xs = torch.where(active[:, None], x[:t].float(), torch.zeros((), device=dev))
            index = torch.arange(t, device=dev)
            cu = ctx.cu_seqlens[:ctx.n_seqs + 1].long()
            seq = torch.searchsorted(cu[1:].contiguous(), index, right=True)   # each token's sequence
            start = cu[seq]
            running = torch.cumsum(xs, 0)
            before = torch.where((start > 0)[:, None], running[(start - 1).clamp(min=0)],
                                 torch.zeros((), device=dev))
            state = entry.state                                       # [slots, hidden + 1]
            mine = state[slots]
            sums = mine[:, :h] + running - before
            counts = mine[:, h] + (index - start + 1)
            out = (sums / counts[:, None]) @ self.w.t()
            if writes_cache:
                last = cu[1:] - 1                                     # the last token of each sequence
                new = torch.cat([sums[last], counts[last, None]], dim=1)
                state.index_copy_(0, slots[last], torch.where(active[last][:, None], new, state[slots[last]]))
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


def toy_greedy(folder, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        out.append(int(plain_logits(folder, ids)[-1].argmax()))
        ids.append(out[-1])
    return out


def test_stateful_mixer_inside_the_captured_decode_step(tmp_path):
    """The toy architecture through ``generate_all`` with the CUDA graph on: the mixer's state is
    advanced inside the captured step by device code only, six requests go through an engine of
    two slots in three batches (a slot's state must start from zero each time), a request with a
    budget of 3 ends while its batch mate goes on.  Tokens against the plain toy model, 32-bit."""
    from enginekernel_b200 import Engine, registry
    from enginekernel_b200.weights import write_random_model
    ToyConfig = define_toy()
    try:
        folder = write_random_model(str(tmp_path / "toy"), ToyConfig.from_dict(RAW), seed=4)
        eng = Engine(folder, "float32", max_tokens=512, max_batch=2, use_graph=True)
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (30, 4, 11, 60, 2, 17)]
        budgets = [20, 20, 3, 20, 20, 12]
        got = eng.generate_all(prompts, budgets)
        want = [toy_greedy(folder, p, n) for p, n in zip(prompts, budgets)]
        assert got == want
        assert max(len(set(w)) for w in want) >= 4        # not one repeated token
        assert eng.cache.book.open_slots() == []
        # the captured step really ran (a graph exists) and the host never laid those steps out
        assert any(st.graph is not None for st in eng.backend._states.values())
        again = eng.generate_all(prompts[::-1], budgets[::-1])
        assert again == want[::-1]
    finally:
        registry.unregister_part("mixer", "running_mean")
        registry.unregister_architecture("ToyMixedForCausalLM")


# -- a layer that sees all keys beside a layer that sees a window of them ----------------------
WINDOW = 100
WINDOW_RAW = {"architectures": ["ToyWindowForCausalLM"], "hidden_size": 72, "vocab_size": 113, "heads": 4,
              "kv_heads": 2, "head_dim": 64, "ff_width": 96, "eps": 1e-6, "theta": 10000.0,
              "window": WINDOW, "max_positions": 1024}


def define_window_toy():
    from enginekernel_b200 import registry
    from enginekernel_b200.config.base import ModelConfig, key
    from enginekernel_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec

    @dataclasses.dataclass(frozen=True)
    class WindowConfig(ModelConfig):
        architecture = "ToyWindowForCausalLM"
        hidden_size: int = key("hidden_size")
        vocab_size: int = key("vocab_size")
        heads: int = key("heads")
        kv_heads: int = key("kv_heads")
        head_dim: int = key("head_dim")
        width: int = key("ff_width")
        eps: float = key("eps")
        theta: float = key("theta")
        window: int = key("window")
        max_positions: int = key("max_positions")

    def build(cfg):
        h = cfg.hidden_size

        def layer(p, window):
            norms = {n: PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": f"{p}.{n}.gain"})
                     for n in ("pre_mixer", "pre_feed_forward")}
            attn = PartSpec("attention", {
                "hidden_size": h, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                "head_dim": cfg.head_dim, "scale": cfg.head_dim ** -0.5, "qk_norm_eps": cfg.eps,
                "window": window,
                "position": PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.theta,
                                                   "rotary_dim": cfg.head_dim})},
                {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "o": f"{p}.o",
                 "q_norm": f"{p}.qn", "k_norm": f"{p}.kn"})
            ff = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": cfg.width},
                          {"gate": f"{p}.ff.gate", "up": f"{p}.ff.up", "down": f"{p}.ff.down"})
            return LayerSpec(PartSpec("pre_norm"), attn, ff, norms)

        return ModelSpec(
            hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
            embedding=TensorSpec("embed", (cfg.vocab_size, h), "embedding"),
            layers=[layer("l0", None), layer("l1", cfg.window), layer("l2", cfg.window)],
            schedule=[RunSpec(0, 0), RunSpec(1, 1), RunSpec(2, 2)],
            final_norm=PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": "final.gain"}),
            lm_head=TensorSpec("head", (cfg.vocab_size, h)))

    registry.register_architecture("ToyWindowForCausalLM", WindowConfig, build, replace=True)
    return WindowConfig


def window_plain_logits(folder, ids, window=WINDOW):
    c = WINDOW_RAW
    w = plain.read_weights(folder, torch.float32)
    s, nh, nkv, d, eps = len(ids), c["heads"], c["kv_heads"], c["head_dim"], c["eps"]
    cos, sin = plain.rope_tables(s, d, c["theta"], torch.float32)
    r = w["embed"][torch.tensor(ids)]
    for p, win in (("l0", None), ("l1", window), ("l2", window)):
        a = plain.rms_norm(r, w[f"{p}.pre_mixer.gain"], eps)
        q = plain.qk_norm_rope((a @ w[f"{p}.q"].t()).view(s, nh, d), w[f"{p}.qn"], cos, sin, eps)
        k = plain.qk_norm_rope((a @ w[f"{p}.k"].t()).view(s, nkv, d), w[f"{p}.kn"], cos, sin, eps)
        v = (a @ w[f"{p}.v"].t()).view(s, nkv, d)
        r = r + plain.causal_gqa_attention(q, k, v, d ** -0.5, window=win) @ w[f"{p}.o"].t()
        m = plain.rms_norm(r, w[f"{p}.pre_feed_forward.gain"], eps)
        g, u = m @ w[f"{p}.ff.gate"].t(), m @ w[f"{p}.ff.up"].t()
        r = r + (torch.nn.functional.silu(g) * u) @ w[f"{p}.ff.down"].t()
    return plain.rms_norm(r, w["final.gain"], eps) @ w["head"].t()


def sharpen_window_toy(folder):
    """Make single keys matter: larger query and key matrices in the windowed layers, so that the
    softmax is peaked and the key at the window's edge carries visible weight."""
    import os
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for name in ("l1.q", "l1.k", "l2.q", "l2.k", "l1.v", "l2.v", "l1.o", "l2.o"):
        tensors[name] = (tensors[name].float() * 6).to(tensors[name].dtype)
    save_file(tensors, path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_through_the_engine(tmp_path, dtype):
    """A model with one layer that sees every key and two that see the last 100: two page groups.
    A 300-token prompt runs in pieces of at most 128 tokens (pages behind the window are given
    back after each piece), then 80 tokens one by one across page boundaries.  The plain model
    with a window of 99 or 101 is far outside the tolerance, so an edge that is off by one shows."""
    from enginekernel_b200 import Engine, registry
    from enginekernel_b200.weights import write_random_model
    WindowConfig = define_window_toy()
    try:
        folder = write_random_model(str(tmp_path / "window"), WindowConfig.from_dict(WINDOW_RAW), seed=6)
        sharpen_window_toy(folder)
        g = torch.Generator().manual_seed(2)
        ids = torch.randint(0, 113, (380,), generator=g).tolist()
        want = window_plain_logits(folder, ids)
        for wrong in (WINDOW - 1, WINDOW + 1):
            assert helpers.rel_err(window_plain_logits(folder, ids, wrong)[WINDOW:], want[WINDOW:]) > \
                20 * helpers.TOL["float32"], "the test would not see a window edge that is off by one"
        eng = Engine(folder, dtype, max_tokens=1024, max_batch=2, max_step_tokens=128)
        groups = {g_.spec.window: g_.page_group for g_ in eng.cache.groups}
        assert set(groups) == {None, WINDOW}
        total = eng.cache.num_pages
        slot = eng.open_sequence()
        rows = [eng.step([(slot, ids[:300], list(range(300)))]).cpu()]
        assert len(groups[None].pages_of(slot)) == 5                  # 300 tokens
        assert len(groups[WINDOW].pages_of(slot)) <= 3                # keys 201.. : pages 3 and 4
        for tok in ids[300:]:
            rows.append(eng.step([(slot, [tok], [0])]).cpu())
            assert len(groups[WINDOW].pages_of(slot)) <= 3
        got = torch.cat(rows, 0)
        assert helpers.rel_err(got, want) <= helpers.TOL[dtype]
        assert len(groups[None].pages_of(slot)) == 6
        eng.close_sequence(slot)
        assert groups[None].pool.available() == total and groups[WINDOW].pool.available() == total
        # a second sequence in the same slot, in a batch with a short one, from a reused slot
        got = helpers.batch_then_steps(eng, [ids[:250], ids[5:40]], [200, 30])
        assert helpers.rel_err(got[0], want[:250]) <= helpers.TOL[dtype]
        # generation through the captured decode step crosses the window's edge while decoding;
        # sampled with a fixed seed so that the tokens vary (greedy repeats one token here)
        if dtype == "float32":
            prompts = [ids[:90], ids[100:130]]
            tokens = eng.generate_all(prompts, 40, temperature=1.0, seed=99)
            for b, (p, t) in enumerate(zip(prompts, tokens)):
                seq, ref = list(p), []
                for step in range(40):
                    row = window_plain_logits(folder, seq)[-1]
                    ref.append(plain.sample_token(row, 1.0, 0, 99, b, step))
                    seq.append(ref[-1])
                assert t == ref
                assert len(set(ref)) >= 8
        assert groups[None].pool.available() == total and groups[WINDOW].pool.available() == total
    finally:
        registry.unregister_architecture("ToyWindowForCausalLM")


# -- a feed-forward with routing and another position encoding ---------------------------------
def define_routed_toy():
    from enginekernel_b200 import registry
    from enginekernel_b200.config.base import ModelConfig, key
    from enginekernel_b200.parts.base import FeedForward, PositionEncoding
    from enginekernel_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec

    class StretchedRope(PositionEncoding):
        """Rotation by (position / stretch) x theta^(-2j/rotary_dim) of the first ``rotary_dim``
        dimensions of a head.  The attention part reads ``cos``, ``sin`` and ``rotary_dim``."""

        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.rotary_dim = int(self.param("rotary_dim"))
            self.cos = self.sin = None

        def prepare(self, max_positions):
            rot = self.rotary_dim
            inv = 1.0 / (float(self.param("theta")) ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
            angles = torch.outer(torch.arange(max_positions, dtype=torch.float32) / float(self.param("stretch")), inv)
            self.cos, self.sin = angles.cos().to(self.device), angles.sin().to(self.device)

    class RoutedFeedForward(FeedForward):
        """Each token goes to the one expert its router scores highest; the expert's output is
        weighted by the router's softmax probability.  Router and softmax in 32-bit."""

        @classmethod
        def tensors(cls, spec):
            h, w, e = spec.params["hidden_size"], spec.params["width"], spec.params["experts"]
            out = [TensorSpec(spec.weights["router"], (e, h))]
            for i in range(e):
                out += [TensorSpec(spec.weights["in"].format(i), (w, h)),
                        TensorSpec(spec.weights["out"].format(i), (h, w))]
            return out

        def load(self, tensors):
            e = self.param("experts")
            self.router = tensors[self.spec.weights["router"]].float()
            self.w_in = [tensors[self.spec.weights["in"].format(i)].float() for i in range(e)]
            self.w_out = [tensors[self.spec.weights["out"].format(i)].float() for i in range(e)]

        def forward(self, x, ctx):
            x = x[:ctx.n_tokens].float()
            prob = torch.softmax(x @ self.router.t(), dim=-1)
            top, choice = prob.max(dim=-1)
            y = torch.zeros_like(x)
            for i in range(len(self.w_in)):
                mine = (choice == i).float()[:, None]       # no host decision: the same work every step
                y += mine * (torch.relu(x @ self.w_in[i].t()) @ self.w_out[i].t())
            return (top[:, None] * y).to(self.dtype)

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        architecture = "ToyRoutedForCausalLM"
        hidden_size: int = key("hidden_size")
        vocab_size: int = key("vocab_size")
        heads: int = key("heads")
        kv_heads: int = key("kv_heads")
        head_dim: int = key("head_dim")
        width: int = key("ff_width")
        experts: int = key("experts")
        eps: float = key("eps")
        theta: float = key("theta")
        stretch: float = key("stretch")
        rotary_dim: int = key("rotary_dim")
        max_positions: int = key("max_positions")

    def build(cfg):
        h = cfg.hidden_size

        def norms(p):
            return {n: PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": f"{p}.{n}.gain"})
                    for n in ("pre_mixer", "pre_feed_forward")}

        def attn(p, position):
            return PartSpec("attention", {
                "hidden_size": h, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                "head_dim": cfg.head_dim, "scale": cfg.head_dim ** -0.5, "qk_norm_eps": None,
                "window": None, "position": position},
                {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "o": f"{p}.o"})

        plain_rope = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.theta,
                                            "rotary_dim": cfg.head_dim})
        stretched = PartSpec("stretched_rope", {"theta": cfg.theta, "rotary_dim": cfg.rotary_dim,
                                                "stretch": cfg.stretch})
        layers = [
            LayerSpec(PartSpec("pre_norm"), attn("l0", plain_rope),
                      PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": cfg.width},
                               {"gate": "l0.ff.gate", "up": "l0.ff.up", "down": "l0.ff.down"}), norms("l0")),
            LayerSpec(PartSpec("pre_norm"), attn("l1", stretched),
                      PartSpec("routed", {"hidden_size": h, "width": cfg.width, "experts": cfg.experts},
                               {"router": "l1.ff.router", "in": "l1.ff.{}.in", "out": "l1.ff.{}.out"}),
                      norms("l1")),
        ]
        return ModelSpec(
            hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
            embedding=TensorSpec("embed", (cfg.vocab_size, h), "embedding"), layers=layers,
            schedule=[RunSpec(0, 0), RunSpec(1, 1)],
            final_norm=PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": "final.gain"}),
            lm_head=TensorSpec("head", (cfg.vocab_size, h)))

    registry.register_part("position", "stretched_rope", StretchedRope, replace=True)
    registry.register_part("feed_forward", "routed", RoutedFeedForward, replace=True)
    registry.register_architecture("ToyRoutedForCausalLM", RoutedConfig, build, replace=True)
    return RoutedConfig


ROUTED_RAW = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "vocab_size": 83, "heads": 6,
              "kv_heads": 2, "head_dim": 32, "ff_width": 40, "experts": 3, "eps": 1e-6, "theta": 500.0,
              "stretch": 2.5, "rotary_dim": 16, "max_positions": 256}


def routed_plain_logits(folder, ids):
    """The routed toy model on one whole sequence in plain 32-bit torch -> (logits, sure): the
    routed feed-forward is the last thing before the head, so a token whose two best experts are
    almost tied (``sure`` False) may differ in its own logits only."""
    c = ROUTED_RAW
    w = plain.read_weights(folder, torch.float32)
    s, nh, nkv, d, eps, rot = len(ids), c["heads"], c["kv_heads"], c["head_dim"], c["eps"], c["rotary_dim"]
    r = w["embed"][torch.tensor(ids)]

    def rotate(x, cos, sin):                       # x [S, heads, D]; the first `rot` dimensions turn
        n = cos.shape[-1]
        a, b, rest = x[..., :n // 2], x[..., n // 2:n], x[..., n:]
        c1, s1 = cos[:, None, :n // 2], sin[:, None, :n // 2]
        return torch.cat((a * c1 - b * s1, b * c1 + a * s1, rest), dim=-1)

    def angles(n, stretch):
        inv = 1.0 / (c["theta"] ** (torch.arange(0, n, 2, dtype=torch.float32) / n))
        f = torch.outer(torch.arange(s, dtype=torch.float32) / stretch, inv)
        f = torch.cat((f, f), dim=-1)
        return f.cos(), f.sin()

    sure = None
    for p, (cos, sin) in (("l0", angles(d, 1.0)), ("l1", angles(rot, c["stretch"]))):
        a = plain.rms_norm(r, w[f"{p}.pre_mixer.gain"], eps)
        q = rotate((a @ w[f"{p}.q"].t()).view(s, nh, d), cos, sin)
        k = rotate((a @ w[f"{p}.k"].t()).view(s, nkv, d), cos, sin)
        v = (a @ w[f"{p}.v"].t()).view(s, nkv, d)
        r = r + plain.causal_gqa_attention(q, k, v, d ** -0.5) @ w[f"{p}.o"].t()
        m = plain.rms_norm(r, w[f"{p}.pre_feed_forward.gain"], eps)
        if p == "l0":
            g, u = m @ w["l0.ff.gate"].t(), m @ w["l0.ff.up"].t()
            r = r + (torch.nn.functional.silu(g) * u) @ w["l0.ff.down"].t()
        else:
            scores = m @ w["l1.ff.router"].t()
            two = scores.topk(2, dim=-1).values
            sure = (two[:, 0] - two[:, 1]) > 0.05 * scores.abs().max()
            best = torch.softmax(scores, dim=-1).topk(2, dim=-1)
            y = torch.stack([torch.relu(m[t] @ w[f"l1.ff.{int(e)}.in"].t()) @ w[f"l1.ff.{int(e)}.out"].t()
                             for t, e in enumerate(best.indices[:, 0])])
            r = r + best.values[:, :1] * y
    assert len(set(best.indices[:, 0].tolist())) > 1 or s < 8      # the router does choose
    return plain.rms_norm(r, w["final.gain"], eps) @ w["head"].t(), sure


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    from enginekernel_b200 import Engine, registry
    from enginekernel_b200.weights import write_random_model
    RoutedConfig = define_routed_toy()
    try:
        folder = write_random_model(str(tmp_path / "routed"), RoutedConfig.from_dict(ROUTED_RAW), seed=9)
        eng = Engine(folder, dtype, max_tokens=1024, max_batch=4)
        g = torch.Generator().manual_seed(1)
        seqs = [torch.randint(0, 83, (n,), generator=g).tolist() for n in (70, 5, 33)]
        wants = [routed_plain_logits(folder, s) for s in seqs]
        assert sum(int(sure.sum()) for _, sure in wants) > 0.8 * sum(len(s) for s in seqs)
        tol = helpers.TOL[dtype]
        for s, (w, sure) in zip(seqs, wants):
            assert helpers.rel_err(helpers.whole(eng, s)[sure], w[sure]) <= tol
            assert helpers.rel_err(helpers.tail_one_by_one(eng, s, 32)[sure], w[sure]) <= tol
        got = helpers.batch_then_steps(eng, seqs, [40, 5, 2])
        for gl, (w, sure) in zip(got, wants):
            assert helpers.rel_err(gl[sure], w[sure]) <= tol
    finally:
        registry.unregister_part("position", "stretched_rope")
        registry.unregister_part("feed_forward", "routed")
        registry.unregister_architecture("ToyRoutedForCausalLM")


# -- learned absolute positions, an embedding multiplier, a logit multiplier --------------------
LEARNED_RAW = {"architectures": ["ToyLearnedForCausalLM"], "hidden_size": 56, "vocab_size": 101, "heads": 2,
               "kv_heads": 1, "head_dim": 32, "ff_width": 72, "eps": 1e-5, "embedding_multiplier": 3.0,
               "logit_multiplier": 0.25, "max_positions": 200}


def define_learned_toy():
    from enginekernel_b200 import registry
    from enginekernel_b200.config.base import ModelConfig, key
    from enginekernel_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec

    @dataclasses.dataclass(frozen=True)
    class LearnedConfig(ModelConfig):
        architecture = "ToyLearnedForCausalLM"
        hidden_size: int = key("hidden_size")
        vocab_size: int = key("vocab_size")
        heads: int = key("heads")
        kv_heads: int = key("kv_heads")
        head_dim: int = key("head_dim")
        width: int = key("ff_width")
        eps: float = key("eps")
        embedding_multiplier: float = key("embedding_multiplier")
        logit_multiplier: float = key("logit_multiplier")
        max_positions: int = key("max_positions")

    def build(cfg):
        h = cfg.hidden_size

        def layer(p):
            norms = {n: PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": f"{p}.{n}.gain"})
                     for n in ("pre_mixer", "pre_feed_forward")}
            attn = PartSpec("attention", {                      # no rotation: positions are learned
                "hidden_size": h, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                "head_dim": cfg.head_dim, "scale": cfg.head_dim ** -0.5, "qk_norm_eps": None,
                "window": None, "position": None},
                {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "o": f"{p}.o"})
            ff = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": cfg.width},
                          {"gate": f"{p}.ff.gate", "up": f"{p}.ff.up", "down": f"{p}.ff.down"})
            return LayerSpec(PartSpec("pre_norm"), attn, ff, norms)

        return ModelSpec(
            hidden_size=h, vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
            embedding=TensorSpec("embed", (cfg.vocab_size, h), "embedding"),
            layers=[layer("l0"), layer("l1")], schedule=[RunSpec(0, 0), RunSpec(1, 1)],
            final_norm=PartSpec("rms_norm", {"size": h, "eps": cfg.eps}, {"gain": "final.gain"}),
            lm_head=TensorSpec("head", (cfg.vocab_size, h)),
            embedding_multiplier=cfg.embedding_multiplier,
            position_table=TensorSpec("positions", (cfg.max_positions, h), "embedding"),
            logit_multiplier=cfg.logit_multiplier)

    registry.register_architecture("ToyLearnedForCausalLM", LearnedConfig, build, replace=True)
    return LearnedConfig


def learned_plain_logits(folder, ids):
    c = LEARNED_RAW
    w = plain.read_weights(folder, torch.float32)
    s, nh, nkv, d, eps = len(ids), c["heads"], c["kv_heads"], c["head_dim"], c["eps"]
    r = w["embed"][torch.tensor(ids)] * c["embedding_multiplier"] + w["positions"][:s]
    for p in ("l0", "l1"):
        a = plain.rms_norm(r, w[f"{p}.pre_mixer.gain"], eps)
        q = (a @ w[f"{p}.q"].t()).view(s, nh, d)
        k = (a @ w[f"{p}.k"].t()).view(s, nkv, d)
        v = (a @ w[f"{p}.v"].t()).view(s, nkv, d)
        r = r + plain.causal_gqa_attention(q, k, v, d ** -0.5) @ w[f"{p}.o"].t()
        m = plain.rms_norm(r, w[f"{p}.pre_feed_forward.gain"], eps)
        g, u = m @ w[f"{p}.ff.gate"].t(), m @ w[f"{p}.ff.up"].t()
        r = r + (torch.nn.functional.silu(g) * u) @ w[f"{p}.ff.down"].t()
    return c["logit_multiplier"] * (plain.rms_norm(r, w["final.gain"], eps) @ w["head"].t())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_learned_positions_and_multipliers_at_the_model_level(tmp_path, dtype):
    """What stands around the blocks is data too: an architecture with learned absolute positions
    (no rotation in its attention), an embedding multiplier and a logit multiplier, registered from
    here.  The positions matter: the same tokens shifted by one position give other logits."""
    from enginekernel_b200 import Engine, registry
    from enginekernel_b200.weights import write_random_model
    LearnedConfig = define_learned_toy()
    try:
        folder = write_random_model(str(tmp_path / "learned"), LearnedConfig.from_dict(LEARNED_RAW), seed=12)
        eng = Engine(folder, dtype, max_tokens=1024, max_batch=4)
        g = torch.Generator().manual_seed(5)
        seqs = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (90, 3, 41)]
        wants = [learned_plain_logits(folder, s) for s in seqs]
        shifted = learned_plain_logits(folder, [seqs[0][0]] + seqs[0])[1:]
        assert helpers.rel_err(shifted, wants[0]) > 5 * helpers.TOL["bfloat16"], "the positions do not matter"
        tol = helpers.TOL[dtype]
        for s, w in zip(seqs, wants):
            assert helpers.rel_err(helpers.whole(eng, s), w) <= tol
            assert helpers.rel_err(helpers.tail_one_by_one(eng, s, 32), w) <= tol
        got = helpers.batch_then_steps(eng, seqs, [60, 2, 41])
        for gl, w in zip(got, wants):
            assert helpers.rel_err(gl, w) <= tol
        if dtype == "float32":                     # through the captured decode step
            tokens = eng.generate_all([s[:20] for s in seqs[::2]], 16, temperature=1.0, seed=3)
            for b, (p, t) in enumerate(zip([s[:20] for s in seqs[::2]], tokens)):
                seq, ref = list(p), []
                for step in range(16):
                    ref.append(plain.sample_token(learned_plain_logits(folder, seq)[-1], 1.0, 0, 3, b, step))
                    seq.append(ref[-1])
                assert t == ref
    finally:
        registry.unregister_architecture("ToyLearnedForCausalLM")


def test_unknown_kinds_are_named():
    from enginekernel_b200 import registry
    with pytest.raises(registry.RegistryError, match="attention"):
        registry.lookup_part("mixer", "no_such_mixer")
