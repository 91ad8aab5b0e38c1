"""Layers of a real model family's width (Qwen3-4B shape, two layers, random weights):
the kernels at the sizes they are tuned for, against the plain implementation."""

import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain
from tests.plain import tiny_models

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 2560, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 20011, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 4096, "tie_word_embeddings": True,
}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return helpers.make_folder(tmp_path_factory.mktemp("family"), CFG, 3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_family_width_ragged_batch(folder, dtype):
    from enginekernel_b200 import Engine
    model = helpers.plain_model(folder)
    eng = Engine(folder, dtype, max_tokens=2048, max_batch=4)
    seqs = tiny_models.random_prompts(CFG, [150, 37, 70], seed=8)
    got = helpers.batch_then_steps(eng, seqs, [140, 30, 70])
    for s, g in zip(seqs, got):
        err = helpers.rel_err(g, plain.logits(model, s))
        assert err <= helpers.TOL[dtype], (dtype, len(s), err)


def tokens_follow_plain(model, prompt, tokens, dtype):
    """32-bit: the plain arg-max.  bfloat16: every emitted token within twice the logits' bound
    of the plain arg-max at its position, teacher-forced on the emitted tokens."""
    if dtype == "float32":
        assert tokens == plain.greedy(model, prompt, len(tokens))
        return
    lg = plain.logits(model, list(prompt) + list(tokens[:-1]))[len(prompt) - 1:]
    scale = lg.abs().max().item()
    for step, (row, tok) in enumerate(zip(lg, tokens)):
        gap = row.max().item() - row[tok].item()
        assert gap <= 2 * helpers.TOL[dtype] * scale, (step, tok, gap, scale)


@pytest.mark.parametrize("dtype,batch", [("float32", 3), ("bfloat16", 3), ("bfloat16", 24)])
def test_family_width_generation_follows_plain(folder, dtype, batch):
    """Generation through the captured decode step at heads of 128: the q/k/v product that
    normalises, rotates and writes the cache itself, the norms carried by the products (3
    sequences) or the norm kernel (24), the TMA-fed decode attention, positions advanced on the
    device - every token against the plain implementation."""
    from enginekernel_b200 import Engine
    model = helpers.plain_model(folder)
    eng = Engine(folder, dtype, max_tokens=batch * 192, max_batch=batch)
    seqs = tiny_models.random_prompts(CFG, [9 + (13 * i) % 80 for i in range(batch)], seed=21)
    got = eng.generate_all(seqs, 24)
    for p, g in zip(seqs, got):
        assert len(g) == 24
        tokens_follow_plain(model, p, g, dtype)
    eng.runner.check_kernels()


@pytest.mark.parametrize("batch", [3, 24])
def test_family_width_eager_decode_equals_the_captured_step(folder, batch):
    """Without the graph each decode step is launched kernel by kernel, and the state advance of
    one step is still in flight when the next step's kernels are queued behind it: the tokens must
    be the captured step's, bit for bit, over many steps."""
    from enginekernel_b200 import Engine
    seqs = tiny_models.random_prompts(CFG, [20 + (11 * i) % 50 for i in range(batch)], seed=5)
    runs = []
    for use_graph in (True, False):
        eng = Engine(folder, "bfloat16", max_tokens=batch * 256, max_batch=batch, use_graph=use_graph)
        runs.append(eng.generate_all(seqs, 64))
        eng.runner.check_kernels()
    assert runs[0] == runs[1]


def test_family_width_two_dozen_sequences(folder):
    """24 sequences decode together: more rows than the deferred norms take, few enough for the
    q/k/v product to do head norm, rotation and cache write itself (heads of 128)."""
    from enginekernel_b200 import Engine
    model = helpers.plain_model(folder)
    eng = Engine(folder, "bfloat16", max_tokens=24 * 128, max_batch=24)
    lens = [5 + (7 * i) % 40 for i in range(24)]
    seqs = tiny_models.random_prompts(CFG, lens, seed=12)
    got = helpers.batch_then_steps(eng, seqs, [n - 3 for n in lens])
    for s, g in zip(seqs, got):
        err = helpers.rel_err(g, plain.logits(model, s))
        assert err <= helpers.TOL["bfloat16"], (len(s), err)


@pytest.mark.parametrize("batch", [3, 24])
def test_family_width_generation_repeats_bit_for_bit(folder, batch):
    """The same prompts twice: the same tokens at every step (sums over K splits, clusters and
    two accumulators are taken in a fixed order; a barrier that let a thread run ahead would show)."""
    from enginekernel_b200 import Engine
    eng = Engine(folder, "bfloat16", max_tokens=batch * 256, max_batch=batch)
    seqs = tiny_models.random_prompts(CFG, [20 + (11 * i) % 50 for i in range(batch)], seed=5)
    runs = [[list(t) for t in eng.generate(seqs, 96)] for _ in range(2)]
    assert runs[0] == runs[1]
    eng.runner.check_kernels()


# The smallest model of the family at its full depth and vocabulary (28 layers, 151,936 tokens),
# 32-bit logits of a batch of 4 against the plain implementation, then the same in bfloat16.
SMALL_FAMILY = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "tie_word_embeddings": True,
}


@pytest.fixture(scope="module")
def small_family(tmp_path_factory):
    folder = helpers.make_folder(tmp_path_factory.mktemp("small_family"), SMALL_FAMILY, 4)
    model = helpers.plain_model(folder)
    seqs = tiny_models.random_prompts(SMALL_FAMILY, [70, 9, 33, 130], seed=3)
    want = [plain.logits(model, s)[-12:] for s in seqs]
    del model
    return folder, seqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_small_family_model_at_full_depth_batch_of_4(small_family, dtype):
    from enginekernel_b200 import Engine
    folder, seqs, want = small_family
    eng = Engine(folder, dtype, max_tokens=4 * 192, max_batch=4)
    got = helpers.batch_then_steps(eng, seqs, [len(s) - 6 for s in seqs])
    for s, g, w in zip(seqs, got, want):
        err = helpers.rel_err(g[-12:] if len(s) >= 12 else g, w[-len(s):])
        assert err <= helpers.TOL[dtype], (dtype, len(s), err)
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("adds_to_stream", [False, True])
def test_prompt_products_on_pairs_of_sms_follow_plain(folder, monkeypatch, adds_to_stream):
    """The prompt path with its products on pairs of SMs: q/k/v with head norm, rotation and cache
    write in the epilogue, gate/up with SwiGLU in the epilogue, and (second run) the two products
    that add to the residual stream as well.  The prompts are cut into pieces, so later pieces and
    the decoded tokens read cache pages that the epilogue wrote.  (A few hundred rows would go to
    the library: the rule that wants the tiles to fill the GPU's pairs is switched off here.)"""
    from enginekernel_b200 import Engine
    from enginekernel_b200.ops import lib, linear
    monkeypatch.setattr(linear, "PAIR_MIN_FILL", 0.0)
    monkeypatch.setattr(linear, "PAIR_ADDS_TO_STREAM", adds_to_stream)
    model = helpers.plain_model(folder)
    eng = Engine(folder, "bfloat16", max_tokens=2048, max_batch=4, max_step_tokens=200)
    seqs = tiny_models.random_prompts(CFG, [300, 70, 129], seed=9)
    with lib.LaunchRecord() as record:
        got = helpers.batch_then_steps(eng, seqs, [290, 66, 129])
    eng.runner.check_kernels()
    names = set(record.names())
    assert any(n.startswith("ek_gemm_pair_qkv_rope") for n in names), names
    assert any(n.startswith("ek_gemm_pair_bf16[19456") for n in names), names        # gate/up with SwiGLU
    assert any(n.startswith("library_addmm") for n in names) == (not adds_to_stream), names
    assert not any("qk_norm_rope_kv" in n or "silu_mul" in n for n in names), names  # their kernels did not run
    for s, g in zip(seqs, got):
        err = helpers.rel_err(g, plain.logits(model, s))
        assert err <= helpers.TOL["bfloat16"], (len(s), err)
