"""How the next token is chosen."""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 is greedy (arg-max, ties to the lowest id - all the reference
    does, engine/ek_model.py:490-493).  Otherwise tokens are drawn from
    softmax(logits / temperature) restricted to the ``top_k`` largest logits (0: all).
    ``seed`` and the sequence's index in the request make the draws reproducible and
    independent of what else shares the batch."""
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0
