"""A decoder assembled from a model description: embedding, scheduled blocks, final
norm, LM head.

Nothing here is specific to an architecture: the :class:`ModelSpec` says which parts make
each layer and in which order layers run (a layer may run twice; a run may read the cache
entry another run wrote).  What the reference writes out by hand for its one model
(engine/ek_model.py:280-334 prefill, 360-416 decode) is one ``forward`` here, used for
prompts and for single tokens alike.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..parts.base import StepContext
from ..parts.spec import CacheSpec, ModelSpec, TensorSpec
from ..registry import lookup_part

_LAYER_ROLES = ("mixer", "feed_forward")


def _part_tensors(role, spec):
    return lookup_part(role, spec.kind).tensors(spec)


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorSpec]:
    """Every checkpoint tensor the model reads, by name (a tied LM head is left out)."""
    out: Dict[str, TensorSpec] = {spec.embedding.name: spec.embedding}
    if spec.lm_head.optional_alias is None:
        out[spec.lm_head.name] = spec.lm_head
    if spec.position_table is not None:
        out[spec.position_table.name] = spec.position_table
    for ts in _part_tensors("norm", spec.final_norm):
        out[ts.name] = ts
    for layer in spec.layers:
        for role in _LAYER_ROLES:
            for ts in _part_tensors(role, getattr(layer, role)):
                out[ts.name] = ts
        for norm in layer.norms.values():
            for ts in _part_tensors("norm", norm):
                out[ts.name] = ts
    return out


def ignorable_tensors(spec: ModelSpec) -> List[str]:
    """Names a checkpoint may hold although the model does not read them."""
    return [spec.lm_head.name] if spec.lm_head.optional_alias is not None else []


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.check()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.blocks = []
        for layer in spec.layers:
            mixer = lookup_part("mixer", layer.mixer.kind)(layer.mixer, dtype, device)
            ff = lookup_part("feed_forward", layer.feed_forward.kind)(layer.feed_forward, dtype, device)
            block_cls = lookup_part("block", layer.block.kind)
            missing = [n for n in block_cls.norm_names(layer.block) if n not in layer.norms]
            if missing:
                raise ValueError(f"block {layer.block.kind!r} needs the norms {missing}")
            norms = {n: lookup_part("norm", s.kind)(s, dtype, device) for n, s in layer.norms.items()}
            self.blocks.append(block_cls(layer.block, dtype, device, mixer, ff, norms))
        self.final_norm = lookup_part("norm", spec.final_norm.kind)(spec.final_norm, dtype, device)
        self.embedding = self.lm_head = self.position_table = None
        self._prepared_for = 0

    # -- weights ---------------------------------------------------------------
    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Bind checkpoint tensors (by name, already on the device) to the parts."""
        s = self.spec
        self.embedding = tensors[s.embedding.name].to(self.dtype).contiguous()
        if s.lm_head.optional_alias is not None:
            self.lm_head = self.embedding            # tied (engine/ek_model.py:134)
        else:
            self.lm_head = tensors[s.lm_head.name].to(self.dtype).contiguous()
        if s.position_table is not None:
            self.position_table = tensors[s.position_table.name].to(self.dtype).contiguous()
        self.final_norm.load(tensors)
        for block in self.blocks:
            block.mixer.load(tensors)
            block.feed_forward.load(tensors)
            for norm in block.norms.values():
                norm.load(tensors)

    def prepare(self, max_positions: int) -> None:
        """Size position tables for sequences of up to ``max_positions`` tokens."""
        if max_positions > self.spec.max_positions:
            raise ValueError(f"{max_positions} positions asked for, the model is limited to "
                             f"{self.spec.max_positions}")
        for block in self.blocks:
            block.mixer.prepare(max_positions)
        self._prepared_for = max_positions

    def cache_entry_specs(self) -> List[Optional[CacheSpec]]:
        """One CacheSpec (or None) per cache entry the schedule names."""
        specs: List[Optional[CacheSpec]] = [None] * self.spec.num_cache_entries()
        for run in self.spec.schedule:
            if run.cache is None:
                continue
            cs = self.blocks[run.layer].mixer.cache_spec()
            if specs[run.cache] is not None and cs is not None \
                    and specs[run.cache].group_key() != cs.group_key():
                raise ValueError(f"cache entry {run.cache} is shared by mixers with different needs")
            specs[run.cache] = cs if cs is not None else specs[run.cache]
        return specs

    def weight_bytes_read_per_step(self, n_tokens: int = 1) -> int:
        """Bytes of weights a step of ``n_tokens`` tokens reads, each once: what every scheduled
        run's parts say they read (a layer that runs twice reads twice), the final norm and the
        LM head.  Embedding rows are left out (a few rows of the table)."""
        total = self.lm_head.numel() * self.lm_head.element_size()
        total += self.final_norm.bytes_read_per_step(n_tokens)
        for run in self.spec.schedule:
            b = self.blocks[run.layer]
            for part in (b.mixer, b.feed_forward, *b.norms.values()):
                total += part.bytes_read_per_step(n_tokens)
        return total

    # -- one step -----------------------------------------------------------------
    def hidden(self, ctx: StepContext, cache):
        """Run every scheduled block; returns (stream, pending) with the last block's
        output not yet added to the stream."""
        t = ctx.n_tokens
        for run in self.spec.schedule:                 # what mixers share between layers of this step
            self.blocks[run.layer].mixer.begin_step(ctx)
        stream = ctx.workspace.get("stream", (t, self.spec.hidden_size), torch.float32)
        kernels.embed(stream, self.embedding, ctx.token_ids, t, scale=self.spec.embedding_multiplier,
                      pos_table=self.position_table, positions=ctx.positions)
        pending = None
        schedule = self.spec.schedule
        for i, run in enumerate(schedule):
            block = self.blocks[run.layer]
            entry = cache.entry(run.cache) if run.cache is not None and \
                block.mixer.cache_spec() is not None else None
            # a block that can leave its last add and the next norm to its own last product is told
            # which norm comes next (none after the last block: the final norm picks rows)
            follower = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            next_norm = getattr(follower, "first_norm", lambda: None)() if follower is not None else None
            if next_norm is not None:
                pending = block.forward(stream, pending, ctx, entry, run.writes_cache, next_norm=next_norm)
            else:
                pending = block.forward(stream, pending, ctx, entry, run.writes_cache)
        return stream, pending

    def logits(self, ctx: StepContext, stream, pending, rows, n_rows: int):
        """32-bit logits [n_rows, vocab] at the stream rows ``rows`` (int32, on device)."""
        if n_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        h = self.final_norm.forward(stream, ctx, add=pending, rows=rows, n_rows=n_rows,
                                    write_back=False)
        out = linear(h, self.lm_head, ctx, "logits", n_rows=n_rows, out_dtype=torch.float32)
        if self.spec.logit_multiplier != 1.0:
            kernels.scale_(out, self.spec.logit_multiplier)
        return out

    def forward(self, ctx: StepContext, cache, rows, n_rows: int):
        stream, pending = self.hidden(ctx, cache)
        return self.logits(ctx, stream, pending, rows, n_rows)
