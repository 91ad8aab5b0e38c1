"""The plain implementation against the reference's recorded outputs and itself."""

import os

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.plain import tiny_models

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("tag", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_outputs(tag, tmp_path):
    gold = torch.load(os.path.join(GOLDEN, tag + ".pt"))
    tiny_models.write_tiny(str(tmp_path), gold["config"], gold["weight_seed"], dtype=torch.float32)
    model = plain.PlainModel(str(tmp_path), torch.float32)
    for prompt, want_p, want_d in zip(gold["prompts"], gold["prefill_logits"], gold["decode_logits"]):
        got = plain.logits(model, prompt)
        scale = want_p.abs().max().item()
        assert (got - want_p).abs().max().item() <= 2e-6 * max(scale, 1.0)
        assert (got - want_d).abs().max().item() <= 2e-6 * max(scale, 1.0)


def test_prefix_independence(tmp_path):
    """Causality: logits at a position do not change when tokens are appended."""
    tiny_models.write_tiny(str(tmp_path), tiny_models.TINY_B, 3, dtype=torch.float32)
    model = plain.PlainModel(str(tmp_path), torch.float32)
    ids = tiny_models.random_prompts(tiny_models.TINY_B, [20], seed=5)[0]
    full = plain.logits(model, ids)
    part = plain.logits(model, ids[:11])
    assert torch.allclose(full[:11], part, atol=1e-5, rtol=0)


def test_attention_window_and_groups():
    torch.manual_seed(0)
    s, nh, nkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(s, nh, d), torch.randn(s, nkv, d), torch.randn(s, nkv, d)
    out = plain.causal_gqa_attention(q, k, v, 0.3).view(s, nh, d)
    # head 3 reads kv head 1; position 0 sees only key 0
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)
    w = plain.causal_gqa_attention(q, k, v, 0.3, window=1).view(s, nh, d)
    assert torch.allclose(w[5, 0], v[5, 0], atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    cos, sin = plain.rope_tables(50, 16, 10000.0, torch.float32)
    x = torch.randn(1, 1, 16)
    ones = torch.ones(16)
    a = plain.qk_norm_rope(x, ones, cos[7:8], sin[7:8], 1e-6)
    b = plain.qk_norm_rope(x, ones, cos[0:1], sin[0:1], 1e-6)
    assert torch.allclose(a.norm(), b.norm(), atol=1e-5)
    y = torch.randn(1, 1, 16)
    def dot(p, q):
        xa = plain.qk_norm_rope(x, ones, cos[p:p + 1], sin[p:p + 1], 1e-6)
        ya = plain.qk_norm_rope(y, ones, cos[q:q + 1], sin[q:q + 1], 1e-6)
        return (xa * ya).sum()
    assert torch.allclose(dot(10, 3), dot(27, 20), atol=1e-4)


def test_philox_known_answer():
    # Random123's published known-answer test for Philox-4x32-10
    assert plain.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert plain.philox4x32((0xffffffff,) * 4, (0xffffffff,) * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]


def test_sampling_rules():
    row = torch.tensor([0.0, 5.0, 1.0, 5.0])
    assert plain.sample_token(row, 0.0, 0, 1, 0, 0) == 1          # ties: lowest index
    draws = [plain.sample_token(row, 1.0, 2, 9, 0, s) for s in range(40)]
    assert set(draws) <= {1, 3} and len(set(draws)) == 2
    assert plain.sample_token(row, 0.7, 0, 3, 2, 5) == plain.sample_token(row, 0.7, 0, 3, 2, 5)
