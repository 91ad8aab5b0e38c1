"""Interfaces of the parts a layer is put together from, and the step context.

A part is built from a :class:`~enginekernel_b200.parts.spec.PartSpec` (its kind, its
sizes and constants, the checkpoint names of its tensors), the engine's dtype and a
device.  It never sees the model's configuration or which model it is in.  Roles:

``norm``          ``forward(stream, ctx, add=None, rows=None, write_back=True) -> y``
``position``      ``prepare(max_positions)``; what a mixer needs to place tokens.  The attention part
                  reads ``cos``, ``sin`` (32-bit, [positions, rotary_dim / 2]) and ``rotary_dim``
``mixer``         ``cache_spec()``, ``forward(x, ctx, entry, writes_cache) -> [T, hidden]``
``feed_forward``  ``forward(x, ctx) -> [T, hidden]``
``block``         ``forward(stream, pending, ctx, entry, writes_cache) -> pending``

``stream`` is the 32-bit residual stream ``[T, hidden]``; ``pending`` is a part's output
that has not been added to the stream yet (the add is folded into the next norm, as the
reference folds it into ``add_rms_norm``, engine/ek_model.py:291-296, 326-334).

A norm may be *deferred*: a part that is told which norm follows it (``defer=(stream, norm)``)
may add its output to the stream itself and return a :class:`DeferredNorm` instead of a
tensor (or None, if it only did the add: the norm is then called with nothing to add), and a
part may be given a :class:`DeferredNorm` instead of normalised activations.
Both are optional: a part says so with ``defers_norm`` / ``takes_deferred_norm`` and a norm
with ``deferrable()``; everything else goes through the norm's own ``forward``.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch

from .spec import CacheSpec, PartSpec, TensorSpec


class Workspace:
    """Named scratch tensors that live as long as the runner and are reused by every
    layer, so a step allocates nothing after its first run at a given size."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[tuple, torch.Tensor] = {}

    def get(self, name: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            grow = max(n, int(buf.numel() * 1.5) if buf is not None else 0)
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n].view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclasses.dataclass
class StepContext:
    """One step's tokens as the kernels see them (all index tensors int32, on device).

    Token t of the step belongs to the sequence in slot ``token_slot[t]`` and stands at
    ``positions[t]`` in it (negative: the row belongs to a finished sequence and is
    skipped).  Sequence b owns tokens ``cu_seqlens[b] .. cu_seqlens[b+1]``.
    """
    n_tokens: int
    n_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_slot: torch.Tensor
    cu_seqlens: torch.Tensor
    is_decode: bool                 # every sequence brings exactly one token
    max_new: int                    # longest run of new tokens of one sequence
    max_context: int                # no sequence is longer than this after the step
    dtype: torch.dtype
    device: torch.device
    workspace: Workspace
    #: Host copies of positions, token_slot and cu_seqlens, for parts written in plain torch (tests,
    #: toy parts).  They exist only in steps that the host lays out (``ModelRunner.step``: prompts,
    #: chunks, single tokens through ``Engine.step``).  Inside the decode step of ``generate`` -
    #: captured once in a CUDA graph and replayed - they are None: positions advance on the device
    #: and the host does not know them.  There a part may use only the device tensors above
    #: (``n_tokens``, ``n_seqs``, ``is_decode``, ``max_new``, ``max_context`` and the workspace are
    #: fixed for a captured step), must skip rows whose position is negative, and must not
    #: allocate or synchronise.
    host_positions: Optional[List[int]] = None
    host_token_slot: Optional[List[int]] = None
    host_cu_seqlens: Optional[List[int]] = None
    #: What parts make once per step and share between layers (filled in ``begin_step``), by a key
    #: of the part's choosing.
    shared: Dict[object, object] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class DeferredNorm:
    """A norm y = gain * x * rsqrt(mean(x^2) + eps) whose work was moved into the matrix
    products around it: the stream already holds x (the add is done), ``scaled`` is
    x * gain rounded to the activation dtype, and ``ss`` [rows, tiles] holds the sums of x^2
    per 128-column tile of the stream.  The product that reads ``scaled`` multiplies row r of
    its 32-bit result by rsqrt(sum(ss[r]) / size + eps): the same y . W^T with the rounding
    taken before the row's scale instead of after it."""
    scaled: torch.Tensor
    ss: torch.Tensor
    tiles: int
    size: int
    eps: float


class Part:
    """Base of all parts."""
    role = ""

    @classmethod
    def tensors(cls, spec: PartSpec) -> List[TensorSpec]:
        """The checkpoint tensors an instance built from ``spec`` reads."""
        return []

    def __init__(self, spec: PartSpec, dtype: torch.dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the tensors named in ``spec.weights`` (already on the device, in their
        stored precision) and keep them in the form the kernels want."""

    def bytes_read_per_step(self, n_tokens: int) -> int:
        """Bytes of this part's weights that a step of ``n_tokens`` tokens has to read, each
        once (what a bandwidth roofline divides by time).  The default counts every tensor the
        part holds; a part that touches only some of its weights (routed experts) says how many."""
        return sum(v.numel() * v.element_size() for v in vars(self).values()
                   if isinstance(v, torch.Tensor))

    def param(self, name: str):
        try:
            return self.spec.params[name]
        except KeyError:
            raise KeyError(f"{type(self).__name__} needs the parameter {name!r}") from None


class Norm(Part):
    role = "norm"

    def deferrable(self):
        """(gain [size] in 32-bit, eps) if this norm is gain * x * rsqrt(mean(x^2) + eps) over
        the whole stream row and so can be a :class:`DeferredNorm`; else None."""
        return None

    def forward(self, stream, ctx: StepContext, add=None, rows=None, n_rows=None,
                write_back=True):
        raise NotImplementedError


class PositionEncoding(Part):
    """A rotary encoding gives, after ``prepare``, ``cos`` and ``sin`` [positions, rotary_dim / 2] in
    32-bit on the device and ``rotary_dim``: dimension j < rotary_dim / 2 of a head turns with
    dimension j + rotary_dim / 2 by the angle whose cosine and sine stand at [position, j]; the
    dimensions from ``rotary_dim`` on pass unchanged.  Any table of angles fits."""
    role = "position"

    def prepare(self, max_positions: int) -> None:
        raise NotImplementedError


class Mixer(Part):
    role = "mixer"
    #: ``forward`` takes a DeferredNorm for ``x`` / takes ``defer=(stream, norm)`` and may return one
    takes_deferred_norm = False
    defers_norm = False

    def cache_spec(self) -> Optional[CacheSpec]:
        """What one cache entry of this mixer holds per sequence (None: nothing)."""
        return None

    def prepare(self, max_positions: int) -> None:
        """Called once the longest position is known (tables and the like)."""

    def begin_step(self, ctx: StepContext) -> None:
        """Called for every scheduled mixer before the step's first kernel: the place for what
        depends on the step's sequences but not on the layer (put it into ``ctx.shared``).
        Kernels launched here are complete before any kernel of the step starts."""

    def forward(self, x, ctx: StepContext, entry, writes_cache: bool):
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"
    takes_deferred_norm = False
    defers_norm = False

    def forward(self, x, ctx: StepContext):
        raise NotImplementedError


class Block(Part):
    """An arrangement of norms, a mixer and a feed-forward around the residual stream."""
    role = "block"

    def __init__(self, spec, dtype, device, mixer: Mixer, feed_forward: FeedForward,
                 norms: Dict[str, Norm]):
        super().__init__(spec, dtype, device)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    @classmethod
    def norm_names(cls, spec: PartSpec) -> List[str]:
        return []

    def first_norm(self) -> Optional[Norm]:
        """The norm that takes the incoming ``pending``, if the block can be handed a
        :class:`DeferredNorm` made for it (then ``forward`` also takes ``next_norm=``); else None."""
        return None

    def forward(self, stream, pending, ctx: StepContext, entry, writes_cache: bool):
        raise NotImplementedError
