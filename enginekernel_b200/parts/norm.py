"""RMSNorm over the residual stream.

y = gain * x * rsqrt(mean(x^2) + eps), in 32-bit, with the preceding residual add folded
in when there is one (engine/ek_kernels.py:89-123; gain is a plain factor, no +1, no
bias).  Parameters: ``size``, ``eps``.  Tensor: ``gain`` [size].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import register_part
from .base import Norm
from .spec import TensorSpec


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    @classmethod
    def tensors(cls, spec):
        return [TensorSpec(spec.weights["gain"], (spec.params["size"],), "gain")]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.size, self.eps = int(self.param("size")), float(self.param("eps"))
        self.gain = None

    def load(self, tensors):
        self.gain = tensors[self.spec.weights["gain"]].to(torch.float32).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return self.gain.numel() * self.gain.element_size()

    def deferrable(self):
        return self.gain, self.eps

    def forward(self, stream, ctx, add=None, rows=None, n_rows=None, write_back=True):
        if n_rows is None:
            n_rows = rows.numel() if rows is not None else ctx.n_tokens
        y = ctx.workspace.get("normed" if rows is None else "normed_rows", (n_rows, self.size),
                              self.dtype)
        kernels.rmsnorm(y, stream, self.gain, self.eps, add=add, rows=rows, n_rows=n_rows,
                        write_back=write_back)
        return y
