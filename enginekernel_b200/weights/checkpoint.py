"""Safetensors checkpoints read by tensor name.

Shards are found as the reference finds them (engine/ek_model.py:45-60): the
``weight_map`` of ``model.safetensors.index.json`` when present, else every
``*.safetensors`` in the folder in sorted order; none is an error.  Unlike the
reference, which fails with a bare ``KeyError`` on the first absent tensor and
checks no shapes (engine/ek_model.py:124-129), the folder is compared with what
the model expects before any tensor is read, and one error lists everything that
is missing, unexpected or of the wrong shape.

Tensors keep their stored precision class: 16-bit floats are held as bfloat16, a
tensor stored in 32-bit floating point stays 32-bit, integer tables become int32.
What a compute path needs beyond that (a 32-bit copy for the 32-bit path) is made
by the part that owns the tensor.
"""

from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterable, Mapping

import torch

from ..parts.spec import TensorSpec


class WeightsError(RuntimeError):
    """A checkpoint does not hold what the model needs."""


_FLOAT_TAGS = {"BF16", "F16", "F32", "F64"}
_INT_TAGS = {"I8", "U8", "I16", "U16", "I32", "U32", "I64", "U64", "BOOL"}


class CheckpointIndex:
    """Names, shapes and dtypes of all tensors of a folder, without their data."""

    def __init__(self, folder: str):
        self.folder = folder
        self.file_of: Dict[str, str] = {}
        self.shape_of: Dict[str, tuple] = {}
        self.dtype_of: Dict[str, str] = {}
        index = os.path.join(folder, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                weight_map = json.load(f)["weight_map"]
            files = sorted(set(weight_map.values()))
        else:
            weight_map = None
            files = sorted(os.path.basename(p) for p in glob.glob(os.path.join(folder, "*.safetensors")))
            if not files:
                raise FileNotFoundError(f"no safetensors under {folder}")
        from safetensors import safe_open
        for fn in files:
            path = os.path.join(folder, fn)
            if not os.path.exists(path):
                raise FileNotFoundError(f"{index} names {fn}, which is not in {folder}")
            with safe_open(path, framework="pt", device="cpu") as f:
                for name in f.keys():
                    if weight_map is not None and weight_map.get(name, fn) != fn:
                        continue
                    sl = f.get_slice(name)
                    self.file_of[name] = fn
                    self.shape_of[name] = tuple(sl.get_shape())
                    self.dtype_of[name] = str(sl.get_dtype())
        if weight_map is not None:
            for name in weight_map:
                if name not in self.file_of:
                    # listed in the index but absent from its shard: reported as missing later
                    pass

    def names(self):
        return self.file_of.keys()


def check_against(index: CheckpointIndex, expected: Mapping[str, TensorSpec],
                  ignorable: Iterable[str] = ()) -> None:
    """Raise one :class:`WeightsError` naming every mismatch between folder and model.

    ``expected`` holds the tensors that must be read (tied tensors whose alias is
    present are left out by the caller); ``ignorable`` are names that may be present
    without being used (a stored copy of a tied tensor).
    """
    ignorable = set(ignorable)
    missing = sorted(n for n in expected if n not in index.file_of)
    unexpected = sorted(n for n in index.file_of if n not in expected and n not in ignorable)
    wrong_shape, wrong_type = [], []
    for name, spec in expected.items():
        if name not in index.file_of:
            continue
        if tuple(index.shape_of[name]) != tuple(spec.shape):
            wrong_shape.append(f"{name}: file has {list(index.shape_of[name])}, "
                               f"model needs {list(spec.shape)}")
        tag = index.dtype_of[name]
        want = _FLOAT_TAGS if spec.numeric == "float" else _INT_TAGS
        if tag not in want:
            wrong_type.append(f"{name}: stored as {tag}, model needs "
                              f"{'a floating-point' if spec.numeric == 'float' else 'an integer'} tensor")
    if not (missing or unexpected or wrong_shape or wrong_type):
        return
    lines = [f"checkpoint {index.folder} does not match the model:"]
    for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                         ("wrong shapes", wrong_shape), ("wrong types", wrong_type)):
        if items:
            lines.append(f"  {title} ({len(items)}):")
            lines.extend(f"    {it}" for it in items)
    raise WeightsError("\n".join(lines))


def stored_class(t: torch.Tensor) -> torch.Tensor:
    """Bring a tensor to the dtype it is kept in (see the module text)."""
    if t.dtype in (torch.float32, torch.bfloat16, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if not t.dtype.is_floating_point:
        return t.to(torch.int32)
    return t.to(torch.bfloat16)


def read_tensors(index: CheckpointIndex, names: Iterable[str], device="cpu") -> Dict[str, torch.Tensor]:
    """Read the named tensors straight to ``device``, one open handle per shard."""
    from safetensors import safe_open
    dev = str(torch.device(device))
    by_file: Dict[str, list] = {}
    for n in names:
        by_file.setdefault(index.file_of[n], []).append(n)
    out: Dict[str, torch.Tensor] = {}
    for fn, group in by_file.items():
        with safe_open(os.path.join(index.folder, fn), framework="pt", device=dev) as f:
            for n in group:
                out[n] = stored_class(f.get_tensor(n))
    return out
