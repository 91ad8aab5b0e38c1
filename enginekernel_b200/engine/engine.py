"""The Python entry point.

``Engine(model_path)`` and ``engine.generate(input_ids, max_new_tokens)`` keep the
reference's names and meaning (engine/engine.py:770-830, 573-634): token ids in, a
generator that yields one list of tokens (one per sequence) per step.  On top of that:
the precision (``dtype``), the cache size, sampling settings, stop tokens,
``generate_all`` for any number of requests, ``step`` for callers that drive the model
token by token, and a random-weights constructor.  There is no second tier to fall back
to: a failure raises.
"""

from __future__ import annotations

from typing import Iterable, Iterator, List, Optional, Sequence

import torch

from ..cache.store import SequenceCache
from ..config.base import ModelConfig
from ..sampling.params import SamplingParams
from .decode import DeviceBackend
from .generate import GenerationLoop
from .loading import load_model, parse_dtype, random_model
from .runner import DEFAULT_MAX_STEP_TOKENS, ModelRunner, StepEntry

DEFAULT_MAX_TOKENS = 65536


def _require_cuda(device):
    if not torch.cuda.is_available():
        raise RuntimeError("enginekernel_b200 needs a CUDA device (NVIDIA B200, sm_100a); "
                           "there is no CPU path")
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"enginekernel_b200 runs on CUDA devices only, not {dev}")
    return dev


class Engine:
    def __init__(self, model_path: Optional[str] = None, dtype="bfloat16", *,
                 max_tokens: int = DEFAULT_MAX_TOKENS, max_batch: int = 64,
                 max_len: Optional[int] = None, device="cuda:0", use_graph: bool = True,
                 max_step_tokens: int = DEFAULT_MAX_STEP_TOKENS, _model=None, _config=None):
        """``model_path``: a folder with ``config.json`` and safetensors files.
        ``max_tokens``: tokens the cache holds over all live sequences (each sequence
        counted in whole pages of 64); ``max_batch``: most sequences in one batch;
        ``max_len``: longest sequence (default: the smaller of ``max_tokens`` and the
        model's position limit); ``max_step_tokens``: the most tokens one pass over the model
        takes (longer prompt batches are cut into pieces)."""
        self.device = _require_cuda(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        if _model is not None:
            self.model, self.config = _model, _config
        else:
            if model_path is None:
                raise ValueError("Engine needs a model folder (or use Engine.from_config)")
            self.model, self.config = load_model(model_path, self.dtype, self.device)
        self.model_path = model_path
        limit = self.model.spec.max_positions
        max_len = min(max_len or limit, limit, max_tokens)
        self.cache = SequenceCache(self.model.cache_entry_specs(), self.dtype, self.device,
                                   max_tokens=max_tokens, max_slots=max(max_batch, 1),
                                   max_len=max_len)
        self.runner = ModelRunner(self.model, self.cache, max_step_tokens=max_step_tokens)
        self.backend = DeviceBackend(self.runner, max_batch, use_graph=use_graph)
        self.loop = GenerationLoop(self.backend)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int = 0, dtype="bfloat16", device="cuda:0",
                    **kw) -> "Engine":
        """An engine over seeded random weights of ``config``'s shape (drawn on the device)."""
        dev = _require_cuda(device)
        torch.cuda.set_device(dev)
        model, config = random_model(config, seed, parse_dtype(dtype), dev)
        return cls(None, dtype, device=device, _model=model, _config=config, **kw)

    # -- generation -----------------------------------------------------------------
    def generate(self, input_ids, max_new_tokens: int, *, temperature: float = 0.0,
                 top_k: int = 0, seed: int = 0,
                 stop_token_ids: Iterable[int] = ()) -> Iterator[List[int]]:
        """Yield, step by step, one new token per sequence (``-1`` once a sequence has
        ended at a stop token).  The sequences form one batch; their prompts may differ
        in length."""
        sampling = SamplingParams(temperature, top_k, seed)
        return self.loop.stream(input_ids, max_new_tokens, sampling, stop_token_ids)

    def generate_all(self, input_ids, max_new_tokens, *, temperature: float = 0.0,
                     top_k: int = 0, seed: int = 0,
                     stop_token_ids: Iterable[int] = ()) -> List[List[int]]:
        """New tokens of every request (a stop token is kept as the last one), however
        many batches that takes."""
        sampling = SamplingParams(temperature, top_k, seed)
        return self.loop.run(input_ids, max_new_tokens, sampling, stop_token_ids)

    # -- driving the model directly ---------------------------------------------------
    def open_sequence(self) -> int:
        return self.cache.open()

    def close_sequence(self, slot: int) -> None:
        torch.cuda.current_stream().synchronize()
        self.cache.close(slot)
        self.runner.check_kernels()

    def step(self, entries: Sequence) -> torch.Tensor:
        """``entries``: (slot, tokens, want) triples or :class:`StepEntry`.  Returns 32-bit
        logits [wanted places, vocab] on the device, the caller's own (a later step does not
        overwrite them)."""
        es = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        return self.runner.step(es).clone()
