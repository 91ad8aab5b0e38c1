"""Rotary position encoding with NeoX pairing (dimension j rotates with j + rot/2).

Angles: position * theta^(-2j/rot) for j < rot/2, computed in 32-bit on the host with the
reference's formula (engine/ek_model.py:164-174) and kept as 32-bit cos/sin tables of
rot/2 columns (the reference stores the doubled table in the model dtype).  Parameters:
``head_dim``, ``theta``, ``rotary_dim`` (<= head_dim; the dimensions past it are left
unrotated).  The rotation itself happens inside the mixer's kernel, which reads the
tables per token position.
"""

from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import PositionEncoding

_TABLES: Dict[tuple, tuple] = {}


@register_part("position", "rope_neox")
class RopeNeox(PositionEncoding):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.head_dim = int(self.param("head_dim"))
        self.theta = float(self.param("theta"))
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim")
        self.cos = self.sin = None
        self.num_positions = 0

    def prepare(self, max_positions: int) -> None:
        key = (str(self.device), self.theta, self.rotary_dim, max_positions)
        if key not in _TABLES:
            rot = self.rotary_dim
            inv = 1.0 / (self.theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
            t = torch.arange(max_positions, dtype=torch.float32)
            freqs = torch.outer(t, inv)
            if len(_TABLES) > 8:
                _TABLES.clear()
            _TABLES[key] = (freqs.cos().to(self.device).contiguous(),
                            freqs.sin().to(self.device).contiguous())
        self.cos, self.sin = _TABLES[key]
        self.num_positions = max_positions
