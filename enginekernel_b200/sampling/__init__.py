"""Sampling: parameters here; the kernel is ``ops.kernels.sample`` (csrc/sampling.cu)."""
from .params import SamplingParams

__all__ = ["SamplingParams"]
