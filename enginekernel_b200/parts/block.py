"""Pre-norm residual block: stream += mixer(norm(stream)); stream += ff(norm(stream)).

The add of a part's output is folded into the norm that follows it, so a block takes the
previous block's not-yet-added output (``pending``) and returns its own
(engine/ek_model.py:291-296, 312, 326-334).  Norms: ``pre_mixer``, ``pre_feed_forward``.
"""

from __future__ import annotations

from ..registry import register_part
from .base import Block, DeferredNorm


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_names(cls, spec):
        return ["pre_mixer", "pre_feed_forward"]

    def first_norm(self):
        """The norm that takes this block's incoming ``pending``, if the part behind it can read
        a deferred norm; else None."""
        return self.norms["pre_mixer"] if self.mixer.takes_deferred_norm else None

    def forward(self, stream, pending, ctx, entry, writes_cache=True, next_norm=None):
        """``next_norm``: the norm that will take the returned ``pending`` (the next block's
        first), or None; with it the feed-forward may return a DeferredNorm."""
        if isinstance(pending, DeferredNorm):
            a = pending                          # made for pre_mixer by the block before
        else:
            a = self.norms["pre_mixer"].forward(stream, ctx, add=pending)
        if self.mixer.defers_norm and self.feed_forward.takes_deferred_norm:
            o = self.mixer.forward(a, ctx, entry, writes_cache,
                                   defer=(stream, self.norms["pre_feed_forward"]))
        else:
            o = self.mixer.forward(a, ctx, entry, writes_cache)
        m = o if isinstance(o, DeferredNorm) else self.norms["pre_feed_forward"].forward(stream, ctx, add=o)
        if self.feed_forward.defers_norm and next_norm is not None:
            return self.feed_forward.forward(m, ctx, defer=(stream, next_norm))
        return self.feed_forward.forward(m, ctx)
