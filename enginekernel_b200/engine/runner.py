"""The step function: run the tokens a step brings, from the cache, and return logits.

``ModelRunner.step(entries)`` takes, for each participating sequence, its slot, its next
tokens (one or many) and the places among them whose logits are wanted.  Tokens of all
sequences are packed without padding; each carries its slot and position, keys and values
are appended to the sequence's pages, and attention for a token covers its own sequence up
to itself.  Whole prompts, chunks of prompts, single decoded tokens and batches of unequal
lengths are therefore one code path; nothing depends on how the tokens were cut into steps
or on what else is in the batch.

The reference has three separate entry points for this - ``prefill`` for a padded
rectangle, ``decode`` for one token per row with a shared length, ``verify`` for several
tokens per row at per-row lengths (engine/ek_model.py:280-334, 360-416, 418-473) - and
returns only the last position's hidden state.
"""

from __future__ import annotations

import array
import dataclasses
from typing import List, Optional, Sequence

import torch

from ..cache.store import SequenceCache
from ..parts.base import StepContext, Workspace
from .model import DecoderModel


class StepError(ValueError):
    """A step that cannot be run: bad slot, bad token, bad index."""


@dataclasses.dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()

    def token_tensor(self) -> torch.Tensor:
        """The tokens as an int64 tensor on the host, converted once (a prompt has thousands)."""
        t = self.__dict__.get("_token_tensor")
        if t is None:
            toks = self.tokens
            if isinstance(toks, torch.Tensor):
                t = toks.to(torch.int64).cpu()
            else:
                try:                               # four times as fast as torch's own way from a list
                    t = torch.frombuffer(array.array("q", toks), dtype=torch.int64).clone() if len(toks) \
                        else torch.empty(0, dtype=torch.int64)
                except (TypeError, OverflowError):
                    t = torch.as_tensor([int(x) for x in toks], dtype=torch.int64)
            self.__dict__["_token_tensor"] = t
        return t


class PlanBuffers:
    """Index tensors of a step: one pinned host block, one device block, one copy."""

    FIELDS = ("token_ids", "positions", "token_slot", "want_rows", "cu_seqlens")

    def __init__(self, device, max_tokens: int, max_seqs: int):
        self.device = torch.device(device)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        sizes = {"token_ids": max_tokens, "positions": max_tokens, "token_slot": max_tokens,
                 "want_rows": max_tokens, "cu_seqlens": max_seqs + 1}
        self.offsets, total = {}, 0
        for f in self.FIELDS:
            self.offsets[f] = total
            total += (sizes[f] + 3) // 4 * 4                      # 16-byte aligned fields
        pin = self.device.type == "cuda"
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=pin)
        self.dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        self.sizes = sizes

    def host_view(self, field):
        o = self.offsets[field]
        return self.host[o:o + self.sizes[field]]

    def dev_view(self, field):
        o = self.offsets[field]
        return self.dev[o:o + self.sizes[field]]

    def upload(self):
        self.dev.copy_(self.host, non_blocking=True)


# Tokens one pass over the model takes at most; a step that brings more is cut into pieces.  Bigger
# pieces fill the GPU better (Qwen3-0.6B shape, 64 prompts of 7,936 tokens: 1,048 ms to the first
# token with pieces of 8,192, 931 ms with 32,768, 920 ms with 65,536, 916 ms with 131,072); the
# workspaces grow with the largest piece that is actually run (about 100 KB a token at the Qwen3-4B shape).
DEFAULT_MAX_STEP_TOKENS = 65536


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: SequenceCache,
                 max_step_tokens: int = DEFAULT_MAX_STEP_TOKENS):
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_step_tokens = max_step_tokens
        self.workspace = Workspace(self.device)
        self.plan: Optional[PlanBuffers] = None
        self._uploaded = None          # event: the last step's host->device copies are done
        if model.dtype == torch.bfloat16:
            from ..ops import kernels
            kernels.split_scratch(self.device)      # exist before any graph capture
            kernels.tc_status(self.device)
        model.prepare(min(cache.max_len, model.spec.max_positions))

    def check_kernels(self) -> None:
        """Raise if a kernel reported a failure (a tensor-core GEMM whose bounded barrier wait
        ran out).  Synchronises the device; called where the host waits anyway."""
        if self.model.dtype == torch.bfloat16 and self.device.type == "cuda":
            from ..ops import kernels
            kernels.check_tc_status(self.device)

    def _plan_for(self, n_tokens: int, n_seqs: int) -> PlanBuffers:
        p = self.plan
        if p is None or p.max_tokens < n_tokens or p.max_seqs < n_seqs:
            if p is not None:
                torch.cuda.current_stream().synchronize()          # its last copy may be in flight
            p = PlanBuffers(self.device, max(n_tokens, 256, p.max_tokens * 2 if p else 0),
                            max(n_seqs, 64, p.max_seqs * 2 if p else 0))
            self.plan = p
        return p

    # ------------------------------------------------------------------
    def check(self, entries: Sequence[StepEntry]) -> None:
        vocab = self.model.spec.vocab_size
        limit = min(self.cache.max_len, self.model.spec.max_positions)
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            length = self.cache.length(e.slot)                       # raises if not open
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot} brings no tokens")
            try:
                ids = e.token_tensor()
            except (ValueError, TypeError, OverflowError) as err:
                raise StepError(f"slot {e.slot}: token ids must be integers ({err})") from None
            low, high = int(ids.min()), int(ids.max())
            if low < 0 or high >= vocab:
                raise StepError(f"token id {low if low < 0 else high} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"wanted place {w} is outside the {len(e.tokens)} tokens "
                                    f"of slot {e.slot}")
            if length + len(e.tokens) > limit:
                raise StepError(f"slot {e.slot} would reach {length + len(e.tokens)} tokens; "
                                f"the limit is {limit}")

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one step; returns 32-bit logits [wanted places, vocab] on the device, in
        the order of the entries and of each entry's ``want``.  The result is a view of the
        runner's workspace: it is valid until the next step (``Engine.step`` hands out a copy)."""
        entries = list(entries)
        self.check(entries)
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32,
                               device=self.device)
        # all-or-nothing on pages: a step that cannot run leaves the cache as it was
        self.cache.reserve_all((e.slot, self.cache.length(e.slot) + len(e.tokens)) for e in entries)
        total = sum(len(e.tokens) for e in entries)
        if total <= self.max_step_tokens:
            return self._run(entries)
        # too many tokens for one pass: cut into pieces; later pieces read what earlier
        # pieces left in the cache
        outs = []
        order = []                                                 # (entry index, want index) per output row
        pieces: List[List[tuple]] = [[]]
        room = self.max_step_tokens
        for i, e in enumerate(entries):
            start = 0
            while start < len(e.tokens):
                if room == 0:
                    pieces.append([])
                    room = self.max_step_tokens
                n = min(room, len(e.tokens) - start)
                pieces[-1].append((i, start, n))
                start += n
                room -= n
        for piece in pieces:
            sub = []
            for i, start, n in piece:
                e = entries[i]
                want = [w - start for w in e.want if start <= w < start + n]
                order += [(i, w) for w in e.want if start <= w < start + n]
                sub.append(StepEntry(e.slot, e.tokens[start:start + n], want))
            outs.append(self._run(sub).clone())
        logits = torch.cat(outs, 0)
        wanted = [(i, w) for i, e in enumerate(entries) for w in e.want]
        if order != wanted:
            index = {pair: r for r, pair in enumerate(order)}
            perm = torch.tensor([index[p] for p in wanted], dtype=torch.long, device=self.device)
            logits = logits.index_select(0, perm)
        return logits

    def _run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        n_tokens = sum(len(e.tokens) for e in entries)
        if self._uploaded is not None:
            self._uploaded.synchronize()   # the pinned buffers are about to be rewritten
        plan = self._plan_for(n_tokens, len(entries))
        ids, pos = plan.host_view("token_ids"), plan.host_view("positions")
        slot, cu = plan.host_view("token_slot"), plan.host_view("cu_seqlens")
        want_rows = plan.host_view("want_rows")
        t = nw = 0
        max_new = max_context = 0
        h_pos, h_slot, h_cu = [], [], [0]
        for b, e in enumerate(entries):
            n = len(e.tokens)
            past = self.cache.length(e.slot)
            ids[t:t + n] = e.token_tensor()
            pos[t:t + n] = torch.arange(past, past + n, dtype=torch.int32)
            slot[t:t + n] = e.slot
            h_pos += range(past, past + n)
            h_slot += [e.slot] * n
            for w in e.want:
                want_rows[nw] = t + int(w)
                nw += 1
            t += n
            cu[b + 1] = t
            h_cu.append(t)
            max_new = max(max_new, n)
            max_context = max(max_context, past + n)
        cu[0] = 0
        plan.upload()
        self.cache.upload_tables()
        if self.device.type == "cuda":
            self._uploaded = self._uploaded or torch.cuda.Event()
            self._uploaded.record()
        ctx = StepContext(
            n_tokens=n_tokens, n_seqs=len(entries), token_ids=plan.dev_view("token_ids"),
            positions=plan.dev_view("positions"), token_slot=plan.dev_view("token_slot"),
            cu_seqlens=plan.dev_view("cu_seqlens"), is_decode=(max_new == 1), max_new=max_new,
            max_context=max_context, dtype=self.model.dtype, device=self.device,
            workspace=self.workspace, host_positions=h_pos, host_token_slot=h_slot,
            host_cu_seqlens=h_cu)
        logits = self.model.forward(ctx, self.cache, plan.dev_view("want_rows"), nw)
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        return logits
