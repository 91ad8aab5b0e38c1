"""Each part of a layer alone against the plain formulas, at sizes of its own."""

import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def bf16_round(t):
    return t.to(torch.bfloat16).float()


def build(role, spec, dtype, tensors):
    from enginekernel_b200.registry import lookup_part
    part = lookup_part(role, spec.kind)(spec, DT[dtype], DEV)
    part.load({k: v.to(torch.bfloat16).to(DEV) for k, v in tensors.items()})
    return part


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rms_norm_part(dtype):
    from enginekernel_b200.parts.spec import PartSpec
    h, t = 176, 9
    gain = 1 + 0.1 * rnd(h, seed=1)
    part = build("norm", PartSpec("rms_norm", {"size": h, "eps": 2e-5}, {"gain": "g"}), dtype, {"g": gain})
    assert [ts.name for ts in type(part).tensors(part.spec)] == ["g"]
    ctx = helpers.make_context(DT[dtype], DEV, list(range(t)), [0] * t, [0, t])
    stream = rnd(t, h, seed=2).to(DEV)
    add = rnd(t, h, seed=3).to(DT[dtype]).to(DEV)
    want_stream = stream.cpu() + add.float().cpu()
    y = part.forward(stream, ctx, add=add)
    want = plain.rms_norm(want_stream, bf16_round(gain), 2e-5)
    assert helpers.rel_err(y, want) <= TOL[dtype]
    assert helpers.rel_err(stream, want_stream) <= 1e-6


def test_rope_part_tables():
    from enginekernel_b200.parts.spec import PartSpec
    from enginekernel_b200.registry import lookup_part
    part = lookup_part("position", "rope_neox")(
        PartSpec("rope_neox", {"head_dim": 48, "theta": 50000.0, "rotary_dim": 48}), torch.float32, DEV)
    part.prepare(300)
    cos, sin = plain.rope_tables(300, 48, 50000.0, torch.float32)
    assert torch.equal(part.cos.cpu(), cos[:, :24]) and torch.equal(part.sin.cpu(), sin[:, :24])
    with pytest.raises(ValueError):
        lookup_part("position", "rope_neox")(
            PartSpec("rope_neox", {"head_dim": 48, "theta": 1.0, "rotary_dim": 50}), torch.float32, DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,d,window", [(4, 2, 32, None), (6, 1, 48, None), (8, 2, 64, 5)])
def test_attention_part(dtype, nh, nkv, d, window):
    """Two sequences of unequal length in one step, then one token each: against the plain
    per-part functions on whole sequences.  With a window the cache group frees pages."""
    from enginekernel_b200.cache import SequenceCache
    from enginekernel_b200.parts.spec import PartSpec
    h, eps, theta = 80, 1e-5, 10000.0
    w = {"q": rnd(nh * d, h, seed=1, scale=0.2), "k": rnd(nkv * d, h, seed=2, scale=0.2),
         "v": rnd(nkv * d, h, seed=3, scale=0.2), "o": rnd(h, nh * d, seed=4, scale=0.2),
         "qn": 1 + 0.1 * rnd(d, seed=5), "kn": 1 + 0.1 * rnd(d, seed=6)}
    spec = PartSpec("attention", {
        "hidden_size": h, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "scale": d ** -0.5,
        "qk_norm_eps": eps, "window": window,
        "position": PartSpec("rope_neox", {"head_dim": d, "theta": theta, "rotary_dim": d})},
        {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "qn", "k_norm": "kn"})
    part = build("mixer", spec, dtype, w)
    part.prepare(256)
    cs = part.cache_spec()
    assert (cs.kind, cs.heads, cs.head_dim, cs.window) == ("kv", nkv, d, window)
    cache = SequenceCache([cs], DT[dtype], DEV, max_tokens=512, max_slots=4)
    lens = [70, 9]
    xs = [rnd(n + 1, h, seed=10 + i) for i, n in enumerate(lens)]
    wr = {k: bf16_round(v) for k, v in w.items()}

    def want(x):
        s = x.shape[0]
        cos, sin = plain.rope_tables(s, d, theta, torch.float32)
        xx = bf16_round(x) if dtype == "bfloat16" else x
        q = plain.qk_norm_rope((xx @ wr["q"].t()).view(s, nh, d), wr["qn"], cos, sin, eps)
        k = plain.qk_norm_rope((xx @ wr["k"].t()).view(s, nkv, d), wr["kn"], cos, sin, eps)
        v = (xx @ wr["v"].t()).view(s, nkv, d)
        return plain.causal_gqa_attention(q, k, v, d ** -0.5, window) @ wr["o"].t()

    wants = [want(x) for x in xs]
    slots = [cache.open(), cache.open()]
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
    cache.upload_tables()
    pos = list(range(lens[0])) + list(range(lens[1]))
    sl = [slots[0]] * lens[0] + [slots[1]] * lens[1]
    ctx = helpers.make_context(DT[dtype], DEV, pos, sl, [0, lens[0], sum(lens)])
    x = torch.cat([xs[0][:lens[0]], xs[1][:lens[1]]]).to(DT[dtype]).to(DEV)
    out = part.forward(x, ctx, cache.entry(0), True)
    assert helpers.rel_err(out[:lens[0]], wants[0][:lens[0]]) <= TOL[dtype]
    assert helpers.rel_err(out[lens[0]:sum(lens)], wants[1][:lens[1]]) <= TOL[dtype]
    for s, n in zip(slots, lens):
        cache.advance(s, n)
        cache.reserve(s, n + 1)
    cache.upload_tables()
    if window:
        assert len(cache.entry(0)._group.page_group.pages_of(slots[0])) == 1   # positions 64.. only
    ctx = helpers.make_context(DT[dtype], DEV, lens, slots, [0, 1, 2])
    x = torch.stack([xs[0][lens[0]], xs[1][lens[1]]]).to(DT[dtype]).to(DEV)
    out = part.forward(x, ctx, cache.entry(0), True)
    assert helpers.rel_err(out[0], wants[0][lens[0]]) <= TOL[dtype]
    assert helpers.rel_err(out[1], wants[1][lens[1]]) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [3, 100])
def test_gated_mlp_part(dtype, rows):
    from enginekernel_b200.parts.spec import PartSpec
    h, inter = 96, 224
    w = {"g": rnd(inter, h, seed=1, scale=0.2), "u": rnd(inter, h, seed=2, scale=0.2),
         "d": rnd(h, inter, seed=3, scale=0.2)}
    spec = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": inter, "activation": "silu"},
                    {"gate": "g", "up": "u", "down": "d"})
    part = build("feed_forward", spec, dtype, w)
    x = rnd(rows, h, seed=4)
    ctx = helpers.make_context(DT[dtype], DEV, list(range(rows)), [0] * rows, [0, rows])
    out = part.forward(x.to(DT[dtype]).to(DEV), ctx)
    xx = bf16_round(x) if dtype == "bfloat16" else x
    named = {"mlp.gate_proj.weight": bf16_round(w["g"]), "mlp.up_proj.weight": bf16_round(w["u"]),
             "mlp.down_proj.weight": bf16_round(w["d"])}
    assert helpers.rel_err(out, plain.swiglu_mlp(xx, named, "")) <= TOL[dtype]
    with pytest.raises(ValueError, match="activation"):
        build("feed_forward", PartSpec("gated_mlp", dict(spec.params, activation="gelu"), spec.weights),
              dtype, w)
