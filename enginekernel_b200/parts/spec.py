"""Plain-data description of a model: which parts, with which sizes, in which order.

An architecture's builder turns its configuration into a :class:`ModelSpec`.
Nothing here holds tensors or launches kernels; the engine instantiates the
registered part classes from it.  The reference has no such layer (its one model
is written out in engine/ek_model.py:280-416); it exists so that layers can differ
from one another and the order of execution is data.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part reads, by its full name in the safetensors files."""
    name: str
    shape: Tuple[int, ...]
    #: how the random-weights mode fills it: "linear" and "embedding" are N(0, std),
    #: "gain" is 1 + N(0, std_gain); "int" tensors are integer tables
    init: str = "linear"
    #: "float" tensors are computed with in the engine's dtype; "int" become int32
    numeric: str = "float"
    #: another tensor name that may stand in when this one is absent (tied weights)
    optional_alias: Optional[str] = None


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` with its sizes and constants in ``params``.

    ``weights`` maps the part's own role names (``"q"``, ``"gate"``, ``"gain"``...)
    to checkpoint tensor names, so no part knows the naming of any model.
    """
    kind: str
    params: Dict[str, object] = dataclasses.field(default_factory=dict)
    weights: Dict[str, str] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and its norms."""
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]


@dataclasses.dataclass(frozen=True)
class RunSpec:
    """One entry of the execution order.

    ``layer`` indexes :attr:`ModelSpec.layers` (a layer may run more than once).
    ``cache`` names the cache entry its mixer uses; two runs naming the same entry
    share it, and a run with ``writes_cache=False`` only reads what another run of
    the same step stored there.
    """
    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: TensorSpec
    layers: List[LayerSpec]
    schedule: List[RunSpec]
    final_norm: PartSpec
    lm_head: TensorSpec            # optional_alias set when tied to the embedding
    #: what goes into the residual stream for token t: embedding[id] * embedding_multiplier, plus
    #: position_table[position] if the model has learned absolute positions ([max_positions, hidden])
    embedding_multiplier: float = 1.0
    position_table: Optional[TensorSpec] = None
    #: logits = logit_multiplier * (final norm . lm_head^T)
    logit_multiplier: float = 1.0

    def num_cache_entries(self) -> int:
        used = [r.cache for r in self.schedule if r.cache is not None]
        return (max(used) + 1) if used else 0

    def check(self) -> None:
        if not self.schedule:
            raise ValueError("a model needs at least one scheduled layer")
        if self.position_table is not None and tuple(self.position_table.shape) != (self.max_positions,
                                                                                     self.hidden_size):
            raise ValueError(f"the position table must be [{self.max_positions}, {self.hidden_size}], "
                             f"not {tuple(self.position_table.shape)}")
        written = set()
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {run.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if run.cache is not None:
                if run.cache < 0:
                    raise ValueError(f"schedule[{i}] names a negative cache entry")
                if run.writes_cache:
                    if run.cache in written:
                        raise ValueError(f"schedule[{i}] writes cache entry {run.cache} "
                                         "that an earlier run already writes")
                    written.add(run.cache)
                elif run.cache not in written:
                    raise ValueError(f"schedule[{i}] reads cache entry {run.cache} "
                                     "before any run wrote it")


@dataclasses.dataclass(frozen=True)
class CacheSpec:
    """What one cache entry of a mixer needs per sequence.

    ``kind="kv"``: keys and values of ``heads`` x ``head_dim`` per token, all of them
    or only the last ``window`` tokens.  ``kind="state"``: one tensor of fixed
    ``shape`` per sequence (32-bit unless ``state_dtype`` says otherwise), zeroed when
    a sequence takes the slot.  Entries with equal specs form one group with storage
    of its own.
    """
    kind: str
    heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    def group_key(self):
        return (self.kind, self.heads, self.head_dim, self.window, self.shape, self.state_dtype)
