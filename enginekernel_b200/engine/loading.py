"""From a model folder (or a configuration and a seed) to a model on the device."""

from __future__ import annotations

import torch

from ..config.base import ModelConfig
from ..registry import config_from_folder, model_spec_for
from ..weights.checkpoint import CheckpointIndex, check_against, read_tensors
from ..weights.random_init import random_tensors
from .model import DecoderModel, expected_tensors, ignorable_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}") from None


def load_model(folder: str, dtype=torch.bfloat16, device="cuda"):
    """Read ``config.json``, pick the architecture from the registry, check the
    checkpoint against what the model needs and load it.  Returns (model, config)."""
    dtype = parse_dtype(dtype)
    config = config_from_folder(folder)
    spec = model_spec_for(config)
    expected = expected_tensors(spec)
    index = CheckpointIndex(folder)
    check_against(index, expected, ignorable_tensors(spec))
    model = DecoderModel(spec, dtype, device)
    model.load(read_tensors(index, expected.keys(), device))
    return model, config


def random_model(config: ModelConfig, seed: int, dtype=torch.bfloat16, device="cuda",
                 stored_dtype=torch.bfloat16):
    """A model with seeded random weights drawn on ``device`` (no folder is written)."""
    dtype = parse_dtype(dtype)
    spec = model_spec_for(config)
    model = DecoderModel(spec, dtype, device)
    model.load(random_tensors(expected_tensors(spec), seed, dtype=stored_dtype, device=device))
    return model, config
