"""Seeded random weights, in memory or written as a model folder.

The reference has no such mode; its tests build a tiny model with an installed
package (bench/test_equivalence.py:19-31).  Distributions: matrices and
embeddings N(0, 0.02), norm gains 1 + N(0, 0.1), drawn tensor by tensor in sorted
name order from one generator, in 32-bit and then rounded to the stored dtype, so a
folder written from (configuration, seed) is the same on every machine when drawn
on the CPU.  Drawing on a GPU (for full-size benchmarks) gives other values.
"""

from __future__ import annotations

import json
import os
from typing import Dict, Mapping

import torch

from ..parts.spec import TensorSpec

LINEAR_STD = 0.02
GAIN_STD = 0.1


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, dtype=torch.bfloat16,
                   device="cpu", vocab_for_int_tables: int = 2) -> Dict[str, torch.Tensor]:
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.numeric == "int":
            out[name] = torch.randint(0, vocab_for_int_tables, spec.shape, generator=gen,
                                      device=dev, dtype=torch.int32)
            continue
        t = torch.randn(spec.shape, generator=gen, device=dev, dtype=torch.float32)
        if spec.init == "gain":
            t.mul_(GAIN_STD).add_(1.0)
        else:
            t.mul_(LINEAR_STD)
        out[name] = t.to(dtype)
    return out


def write_random_model(folder: str, config, seed: int, dtype=torch.bfloat16, device="cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` under ``folder``.  Drawn on
    ``device`` (a GPU is much faster for gigabytes of weights, but gives other values than the CPU)."""
    from safetensors.torch import save_file
    from ..engine.model import expected_tensors
    from ..registry import model_spec_for
    os.makedirs(folder, exist_ok=True)
    spec = model_spec_for(config)
    tensors = random_tensors(expected_tensors(spec), seed, dtype=dtype, device=device)
    tensors = {k: v.cpu() for k, v in tensors.items()}
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, str(dtype))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    save_file({k: v.contiguous() for k, v in tensors.items()},
              os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
