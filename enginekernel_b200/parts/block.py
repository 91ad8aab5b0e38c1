"""Pre-norm residual block: stream += mixer(norm(stream)); stream += ff(norm(stream)).

The add of a part's output is folded into the norm that follows it, so a block takes the
previous block's not-yet-added output (``pending``) and returns its own
(engine/ek_model.py:291-296, 312, 326-334).  Norms: ``pre_mixer``, ``pre_feed_forward``.
"""

from __future__ import annotations

from ..registry import register_part
from .base import Block


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_names(cls, spec):
        return ["pre_mixer", "pre_feed_forward"]

    def forward(self, stream, pending, ctx, entry, writes_cache=True):
        a = self.norms["pre_mixer"].forward(stream, ctx, add=pending)
        o = self.mixer.forward(a, ctx, entry, writes_cache)
        m = self.norms["pre_feed_forward"].forward(stream, ctx, add=o)
        return self.feed_forward.forward(m, ctx)
