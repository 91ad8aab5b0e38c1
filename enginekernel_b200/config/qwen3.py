"""Configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Keys and defaults follow the reference's reader (engine/ek_model.py:26-42):
``head_dim`` falls back to ``hidden_size // num_attention_heads``,
``rms_norm_eps`` to 1e-6, ``rope_theta`` to 10000.0, ``tie_word_embeddings`` to
false and ``max_position_embeddings`` to 32768.  Keys the reference never reads
(``hidden_act``, ``attention_bias``, ``sliding_window``, ``rope_scaling``) are
fixed behaviour here as there: SiLU, no bias, full attention, plain NeoX rotation.
A file that asks for something else in those keys is refused rather than run wrong.
"""

from __future__ import annotations

import dataclasses

from .base import ConfigError, ModelConfig, key


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    architecture = "Qwen3ForCausalLM"

    num_hidden_layers: int = key("num_hidden_layers")
    hidden_size: int = key("hidden_size")
    num_attention_heads: int = key("num_attention_heads")
    num_key_value_heads: int = key("num_key_value_heads")
    head_dim: int = key("head_dim")          # derived when the file leaves it out
    intermediate_size: int = key("intermediate_size")
    vocab_size: int = key("vocab_size")
    rope_theta: float = key("rope_theta", 10000.0)
    rms_norm_eps: float = key("rms_norm_eps", 1e-6)
    max_position_embeddings: int = key("max_position_embeddings", 32768)
    tie_word_embeddings: bool = key("tie_word_embeddings", False)

    @classmethod
    def _derive_missing(cls, field_name, raw):
        if field_name == "head_dim":
            h, n = raw.get("hidden_size"), raw.get("num_attention_heads")
            if isinstance(h, int) and isinstance(n, int) and n > 0:
                if h % n:
                    raise ConfigError("config.json has no head_dim and hidden_size "
                                      f"{h} is not a multiple of num_attention_heads {n}")
                return h // n
        return None

    @classmethod
    def from_dict(cls, raw):
        _refuse_unsupported(raw)
        return super().from_dict(raw)

    def validate(self) -> None:
        for name in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "intermediate_size",
                     "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotate-half RoPE")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")

    # sizes derived as the reference derives them (engine/ek_model.py:41-42)
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads


def _refuse_unsupported(raw: dict) -> None:
    """Options outside the dense decoder that the reference implements."""
    act = raw.get("hidden_act")
    if act is not None and act != "silu":
        raise ConfigError(f"hidden_act {act!r} is not supported (the MLP is SwiGLU with SiLU)")
    if raw.get("attention_bias"):
        raise ConfigError("attention_bias=true is not supported (projections carry no bias)")
    if raw.get("use_sliding_window"):
        raise ConfigError("use_sliding_window=true is not supported (every layer attends to all keys)")
    scaling = raw.get("rope_scaling")
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
        if kind not in (None, "default"):
            raise ConfigError(f"rope_scaling {kind!r} is not supported (plain NeoX rotation only)")
