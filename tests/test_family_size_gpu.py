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
    steps = list(eng.generate(seqs, 5))
    if dtype == "float32":
        assert [[st[b] for st in steps] for b in range(3)] == [plain.greedy(model, s, 5) for s in seqs]


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
