"""The generation loop: requests -> batches -> prefill -> decode steps -> token lists.

Pure host logic over a small backend interface, so its decisions are tested without a
GPU.  A *batch* is a set of requests that start together: their prompts (of unequal
lengths) run in one prefill step, then every sequence gets one token per step.  A
sequence ends at a stop token (which is kept as its last token), or after its
``max_new_tokens``; the batch ends when its last sequence does, its slots are given back
and the next batch starts, until every request is served.

The reference's loop (engine/engine.py:573-634) runs one batch for exactly
``max_new_tokens`` steps with no stop condition and yields one list of tokens per step;
``stream`` keeps that shape.

Backend interface::

    backend.max_batch                     -> int, most sequences in one batch
    backend.token_capacity()              -> int, tokens the cache can hold now
    backend.tokens_needed(prompt_len, n)  -> int, what one request takes of that
    backend.start(prompts, max_new, sampling, stop_ids, streams) -> run
    run.next_tokens() -> list[int]   one token per sequence for the next step
                                     (-1 for a sequence that ended earlier)
    run.close()                           gives the batch's slots back
"""

from __future__ import annotations

import dataclasses
from typing import Iterable, Iterator, List, Optional, Sequence

from ..sampling.params import SamplingParams


class GenerationError(ValueError):
    pass


@dataclasses.dataclass
class Request:
    index: int
    prompt: List[int]
    max_new_tokens: int


def as_rows(input_ids) -> List[List[int]]:
    """Lists, tuples, numpy arrays or tensors -> list of lists of ints
    (engine/engine.py:113-117)."""
    if hasattr(input_ids, "tolist"):
        input_ids = input_ids.tolist()
    rows = [r.tolist() if hasattr(r, "tolist") else [int(t) for t in r] for r in input_ids]
    return [[int(t) for t in r] for r in rows]


class GenerationLoop:
    def __init__(self, backend):
        self.backend = backend

    # -- decisions --------------------------------------------------------------
    def make_requests(self, prompts, max_new_tokens) -> List[Request]:
        rows = as_rows(prompts)
        if isinstance(max_new_tokens, int):
            max_new = [max_new_tokens] * len(rows)
        else:
            max_new = [int(n) for n in max_new_tokens]
            if len(max_new) != len(rows):
                raise GenerationError("max_new_tokens must be one number or one per prompt")
        for i, (r, n) in enumerate(zip(rows, max_new)):
            if not r:
                raise GenerationError(f"prompt {i} is empty")
            if n < 0:
                raise GenerationError(f"max_new_tokens of prompt {i} is negative")
        return [Request(i, r, n) for i, (r, n) in enumerate(zip(rows, max_new))]

    def plan_batches(self, requests: Sequence[Request]) -> List[List[Request]]:
        """Requests in order; a batch closes when the next request would exceed the batch
        limit or the cache.  Each batch starts with the whole cache free."""
        capacity = self.backend.token_capacity()
        batches: List[List[Request]] = []
        current: List[Request] = []
        used = 0
        for r in requests:
            if r.max_new_tokens == 0:
                continue
            need = self.backend.tokens_needed(len(r.prompt), r.max_new_tokens)
            if need > capacity:
                raise GenerationError(
                    f"request {r.index} needs room for {need} tokens "
                    f"({len(r.prompt)} prompt + {r.max_new_tokens} new), the cache holds {capacity}")
            if current and (len(current) >= self.backend.max_batch or used + need > capacity):
                batches.append(current)
                current, used = [], 0
            current.append(r)
            used += need
        if current:
            batches.append(current)
        return batches

    # -- running ------------------------------------------------------------------
    def _run_batch(self, batch: Sequence[Request], sampling, stop_ids) -> Iterator[List[int]]:
        """Yields one list per step with a token per sequence (-1: ended earlier)."""
        stop = set(stop_ids)
        run = self.backend.start([r.prompt for r in batch], [r.max_new_tokens for r in batch],
                                 sampling, sorted(stop), [r.index for r in batch])
        try:
            done = [False] * len(batch)
            count = [0] * len(batch)
            while not all(done):
                toks = [int(t) for t in run.next_tokens()]
                if len(toks) != len(batch):
                    raise GenerationError("the backend returned a step of the wrong width")
                out = []
                for b, t in enumerate(toks):
                    if done[b] or t < 0:
                        if not done[b]:
                            raise GenerationError(f"sequence {batch[b].index} stopped without a reason")
                        out.append(-1)
                        continue
                    count[b] += 1
                    out.append(t)
                    if t in stop or count[b] >= batch[b].max_new_tokens:
                        done[b] = True
                yield out
        finally:
            run.close()

    def run(self, prompts, max_new_tokens, sampling: Optional[SamplingParams] = None,
            stop_token_ids: Iterable[int] = ()) -> List[List[int]]:
        """Serve every request, batch after batch; returns each request's new tokens
        (a stop token included, nothing after it)."""
        sampling = sampling or SamplingParams()
        stop_ids = [int(s) for s in stop_token_ids]
        requests = self.make_requests(prompts, max_new_tokens)
        outputs: List[List[int]] = [[] for _ in requests]
        for batch in self.plan_batches(requests):
            for step in self._run_batch(batch, sampling, stop_ids):
                for r, t in zip(batch, step):
                    if t >= 0:
                        outputs[r.index].append(t)
        return outputs

    def stream(self, prompts, max_new_tokens: int, sampling: Optional[SamplingParams] = None,
               stop_token_ids: Iterable[int] = ()) -> Iterator[List[int]]:
        """One batch, one list of tokens per step as the reference yields them; the
        requests must fit a single batch."""
        sampling = sampling or SamplingParams()
        requests = self.make_requests(prompts, int(max_new_tokens))
        batches = self.plan_batches(requests)
        if len(batches) > 1:
            raise GenerationError(
                f"{len(requests)} requests do not fit one batch (limit {self.backend.max_batch} "
                f"sequences, {self.backend.token_capacity()} tokens); use generate_all")
        if batches:
            yield from self._run_batch(batches[0], sampling, [int(s) for s in stop_token_ids])
