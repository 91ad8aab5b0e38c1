"""Tiny Qwen3 configurations for tests, and a model-folder writer of the tests' own.

A and B differ in every size and option: layers, width, heads and groups, head size
(in B heads x head size differs from the width), MLP width, vocabulary, rotation
base, norm eps, position limit, tied or separate head.  The writer uses only torch
and safetensors so that test inputs do not depend on the package under test.
"""

from __future__ import annotations

import json
import os

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 128, "tie_word_embeddings": True,
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 224,
    "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "max_position_embeddings": 256, "tie_word_embeddings": False,
}

# A third shape for longer runs: one KV head per four query heads, odd sizes.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 176,
    "vocab_size": 331, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "max_position_embeddings": 1024, "tie_word_embeddings": True,
}

# A fourth shape whose head size (64) and group (3 query heads a KV head, which does not divide
# 128) send attention to the TMA-fed decode kernel and the mma.sync prompt kernel; with
# num_key_value_heads = 3 -> group 2 it would take the tcgen05 prompt kernel (TINY_E).
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 200,
    "vocab_size": 413, "rope_theta": 20000.0, "rms_norm_eps": 2e-6,
    "max_position_embeddings": 2048, "tie_word_embeddings": False,
}

# Head size 64, two query heads a KV head: the tcgen05 prompt kernel and the TMA-fed decode kernel.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 104, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 160,
    "vocab_size": 277, "rope_theta": 300000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 2048, "tie_word_embeddings": True,
}


def tensor_shapes(cfg):
    h, nh, nkv, d = (cfg["hidden_size"], cfg["num_attention_heads"],
                     cfg["num_key_value_heads"], cfg["head_dim"])
    i, v = cfg["intermediate_size"], cfg["vocab_size"]
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (v, h)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        shapes.update({
            p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
            p + "self_attn.q_proj.weight": (nh * d, h), p + "self_attn.k_proj.weight": (nkv * d, h),
            p + "self_attn.v_proj.weight": (nkv * d, h), p + "self_attn.o_proj.weight": (h, nh * d),
            p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
            p + "mlp.gate_proj.weight": (i, h), p + "mlp.up_proj.weight": (i, h),
            p + "mlp.down_proj.weight": (h, i)})
    return shapes


def make_tensors(cfg, seed, dtype=torch.bfloat16, linear_std=0.02, gain_std=0.1):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        is_gain = name.endswith("norm.weight") or name.endswith("layernorm.weight")
        out[name] = (1.0 + gain_std * t if is_gain else linear_std * t).to(dtype)
    return out


def write_folder(folder, cfg, tensors):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in tensors.items()},
              os.path.join(folder, "model.safetensors"))
    return folder


def write_tiny(folder, cfg, seed, dtype=torch.bfloat16, **kw):
    return write_folder(folder, cfg, make_tensors(cfg, seed, dtype, **kw))


def random_prompts(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
