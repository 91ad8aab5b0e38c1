"""Configuration, registry, checkpoint errors and the random-weights mode (no GPU)."""

import json
import os

import pytest
import torch

from enginekernel_b200 import registry
from enginekernel_b200.config import ConfigError, Qwen3Config
from enginekernel_b200.engine.model import expected_tensors, ignorable_tensors
from enginekernel_b200.weights import (CheckpointIndex, WeightsError, check_against, read_tensors,
                                       write_random_model)
from tests.plain import tiny_models


def test_config_reads_every_key_and_defaults():
    c = Qwen3Config.from_dict(tiny_models.TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size) == (3, 96, 6, 3, 32, 224, 384)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.q_size == 192 and c.kv_size == 96 and c.group_size == 2
    minimal = {k: tiny_models.TINY_A[k] for k in (
        "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
        "intermediate_size", "vocab_size")}
    d = Qwen3Config.from_dict(minimal)
    # defaults of the reference's reader: engine/ek_model.py:34-40
    assert d.head_dim == 16 and d.rms_norm_eps == 1e-6 and d.rope_theta == 10000.0
    assert d.tie_word_embeddings is False and d.max_position_embeddings == 32768
    assert Qwen3Config.from_dict(d.to_dict()) == d


@pytest.mark.parametrize("change,word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_hidden_layers": 2.5}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding"),
    ({"attention_bias": True}, "bias"),
])
def test_config_errors(change, word):
    raw = dict(tiny_models.TINY_A)
    for k, v in change.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(raw)


def test_registry_by_architecture_name(tmp_path):
    assert "Qwen3ForCausalLM" in registry.architectures()
    with open(tmp_path / "config.json", "w") as f:
        json.dump(tiny_models.TINY_A, f)
    assert isinstance(registry.config_from_folder(str(tmp_path)), Qwen3Config)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(dict(tiny_models.TINY_A, architectures=["NoSuchModel"]), f)
    with pytest.raises(registry.RegistryError, match="Qwen3ForCausalLM"):
        registry.config_from_folder(str(tmp_path))
    with open(tmp_path / "config.json", "w") as f:
        json.dump({k: v for k, v in tiny_models.TINY_A.items() if k != "architectures"}, f)
    with pytest.raises(ConfigError, match="architectures"):
        registry.config_from_folder(str(tmp_path))
    with pytest.raises(ConfigError, match="no config.json"):
        registry.config_from_folder(str(tmp_path / "absent"))


def test_model_description_is_data():
    cfg = Qwen3Config.from_dict(tiny_models.TINY_B)
    spec = registry.model_spec_for(cfg)
    assert [r.layer for r in spec.schedule] == [0, 1, 2] and spec.num_cache_entries() == 3
    assert spec.layers[1].mixer.kind == "attention" and spec.layers[1].feed_forward.kind == "gated_mlp"
    assert spec.layers[0].mixer.params["scale"] == 32 ** -0.5
    names = expected_tensors(spec)
    assert set(names) == set(tiny_models.tensor_shapes(tiny_models.TINY_B))
    for n, shape in tiny_models.tensor_shapes(tiny_models.TINY_B).items():
        assert tuple(names[n].shape) == tuple(shape)
    tied = registry.model_spec_for(Qwen3Config.from_dict(tiny_models.TINY_A))
    assert "lm_head.weight" not in expected_tensors(tied)
    assert ignorable_tensors(tied) == ["lm_head.weight"]


def _index_and_expected(folder, cfg):
    spec = registry.model_spec_for(Qwen3Config.from_dict(cfg))
    return CheckpointIndex(str(folder)), expected_tensors(spec), ignorable_tensors(spec)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny_models.TINY_B
    t = tiny_models.make_tensors(cfg, 0)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(31, dtype=torch.bfloat16)
    t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(96, 97, dtype=torch.bfloat16)
    t["model.layers.0.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int64)
    tiny_models.write_folder(str(tmp_path), cfg, t)
    index, expected, ignorable = _index_and_expected(tmp_path, cfg)
    with pytest.raises(WeightsError) as e:
        check_against(index, expected, ignorable)
    msg = str(e.value)
    for piece in ("missing tensors (2)", "model.layers.1.mlp.up_proj.weight", "model.norm.weight",
                  "unexpected tensors (1)", "model.layers.7.extra.weight", "wrong shapes (2)",
                  "q_norm.weight: file has [31], model needs [32]", "[96, 97]",
                  "wrong types (1)", "input_layernorm.weight: stored as I64"):
        assert piece in msg, piece


def test_untied_model_needs_lm_head_and_tied_model_ignores_it(tmp_path):
    cfg = tiny_models.TINY_B
    t = tiny_models.make_tensors(cfg, 0)
    del t["lm_head.weight"]
    tiny_models.write_folder(str(tmp_path / "b"), cfg, t)
    index, expected, ignorable = _index_and_expected(tmp_path / "b", cfg)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        check_against(index, expected, ignorable)
    cfg = tiny_models.TINY_A
    t = tiny_models.make_tensors(cfg, 0)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    tiny_models.write_folder(str(tmp_path / "a"), cfg, t)
    index, expected, ignorable = _index_and_expected(tmp_path / "a", cfg)
    check_against(index, expected, ignorable)


def test_no_safetensors_and_sharded_index(tmp_path):
    os.makedirs(tmp_path / "empty")
    with pytest.raises(FileNotFoundError, match="no safetensors"):
        CheckpointIndex(str(tmp_path / "empty"))
    # two shards with an index file, as large checkpoints come (engine/ek_model.py:45-49)
    from safetensors.torch import save_file
    cfg = tiny_models.TINY_A
    t = tiny_models.make_tensors(cfg, 0)
    names = sorted(t)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half],
              "model-00002-of-00002.safetensors": names[half:]}
    folder = tmp_path / "sharded"
    os.makedirs(folder)
    for fn, ns in shards.items():
        save_file({n: t[n] for n in ns}, str(folder / fn))
    with open(folder / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {n: fn for fn, ns in shards.items() for n in ns}}, f)
    index, expected, ignorable = _index_and_expected(folder, cfg)
    check_against(index, expected, ignorable)
    got = read_tensors(index, expected.keys())
    assert all(torch.equal(got[n], t[n]) for n in names)


def test_stored_precision_is_kept(tmp_path):
    cfg = tiny_models.TINY_A
    t = tiny_models.make_tensors(cfg, 0)
    t["model.norm.weight"] = t["model.norm.weight"].float()
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].half()
    tiny_models.write_folder(str(tmp_path), cfg, t)
    index, expected, _ = _index_and_expected(tmp_path, cfg)
    got = read_tensors(index, expected.keys())
    assert got["model.norm.weight"].dtype == torch.float32             # 32-bit stays 32-bit
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = Qwen3Config.from_dict(tiny_models.TINY_B)
    a = write_random_model(str(tmp_path / "a"), cfg, seed=5)
    b = write_random_model(str(tmp_path / "b"), cfg, seed=5)
    c = write_random_model(str(tmp_path / "c"), cfg, seed=6)
    assert registry.config_from_folder(a) == cfg
    index, expected, ignorable = _index_and_expected(a, tiny_models.TINY_B)
    check_against(index, expected, ignorable)
    ta, tb, tc = (read_tensors(CheckpointIndex(p), expected.keys()) for p in (a, b, c))
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    assert any(not torch.equal(ta[n], tc[n]) for n in ta)
    w = ta["model.layers.0.mlp.gate_proj.weight"].float()
    g = ta["model.layers.1.input_layernorm.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    assert abs(g.mean().item() - 1.0) < 0.05 and 0.05 < g.std().item() < 0.15
    assert all(v.dtype == torch.bfloat16 for v in ta.values())
    # the plain implementation reads the same folder
    from tests.plain import qwen3_plain as plain
    m = plain.PlainModel(a, torch.float32)
    assert plain.logits(m, [1, 2, 3]).shape == (3, 384)
