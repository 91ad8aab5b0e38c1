"""Qwen3 dense decoder: configuration -> model description.

Layer by layer the reference computes (engine/ek_model.py:280-334, 360-416):
pre-norm residual blocks; grouped-query attention with a per-head RMSNorm on
queries and keys before a NeoX rotation over the whole head; a SwiGLU MLP; a
final RMSNorm and a tied or separate LM head.  Tensor names are the checkpoint's
(engine/ek_model.py:132-159).  This module only names parts and sizes; the parts
themselves know nothing of Qwen3.
"""

from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunSpec, TensorSpec
from ..registry import register_architecture


def build_qwen3(cfg: Qwen3Config) -> ModelSpec:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        rope = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                      "rotary_dim": cfg.head_dim})
        mixer = PartSpec(
            "attention",
            {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
             "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
             "scale": cfg.head_dim ** -0.5,      # engine/ek_model.py:71
             "qk_norm_eps": cfg.rms_norm_eps,    # same key as the layer norms (ek_kernels.py:1127)
             "window": None, "position": rope},
            {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
             "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight",
             "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight"})
        ffn = PartSpec(
            "gated_mlp",
            {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
             "activation": "silu"},
            {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
             "down": p + "mlp.down_proj.weight"})
        norms = {
            "pre_mixer": PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                  {"gain": p + "input_layernorm.weight"}),
            "pre_feed_forward": PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                         {"gain": p + "post_attention_layernorm.weight"}),
        }
        layers.append(LayerSpec(PartSpec("pre_norm"), mixer, ffn, norms))

    embedding = TensorSpec("model.embed_tokens.weight", (cfg.vocab_size, cfg.hidden_size), "embedding")
    lm_head = TensorSpec("lm_head.weight", (cfg.vocab_size, cfg.hidden_size), "linear",
                         optional_alias=embedding.name if cfg.tie_word_embeddings else None)
    spec = ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=embedding, layers=layers,
        schedule=[RunSpec(i, i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                            {"gain": "model.norm.weight"}),
        lm_head=lm_head)
    spec.check()
    return spec


register_architecture(Qwen3Config.architecture, Qwen3Config, build_qwen3)
