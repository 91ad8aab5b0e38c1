"""enginekernel_b200: a small model library with generation for one NVIDIA B200.

Everything between a request's tokens and its next token for the Qwen3 dense decoder:
typed configuration and registry, safetensors weights, layers put together from parts,
a paged cache with a slot per sequence, one step function, a generation loop, sampling,
hand-written CUDA kernels for sm_100a, a true 32-bit path and a trace-replay tool.
"""

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "StepEntry", "load_model", "random_model"):
        from . import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    if name in ("register_architecture", "register_part", "architectures"):
        from . import registry as _r
        return getattr(_r, name)
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)
