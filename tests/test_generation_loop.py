"""The generation loop's decisions, over a scripted backend (no GPU)."""

import pytest

from enginekernel_b200.engine.generate import GenerationError, GenerationLoop, as_rows
from enginekernel_b200.sampling import SamplingParams


class ScriptedRun:
    """Sequence b emits prompt[-1]+1, +2, ... ; stops are the loop's business, but a row
    that ended (stop token or budget) yields -1 afterwards, as the device backend does."""

    def __init__(self, backend, prompts, max_new, stop_ids):
        self.b = backend
        self.next = [p[-1] + 1 for p in prompts]
        self.left = list(max_new)
        self.stop = set(stop_ids)
        self.alive = [True] * len(prompts)
        self.closed = False

    def next_tokens(self):
        self.b.steps += 1
        out = []
        for i in range(len(self.next)):
            if not self.alive[i]:
                out.append(-1)
                continue
            t = self.next[i]
            self.next[i] += 1
            self.left[i] -= 1
            if t in self.stop or self.left[i] <= 0:
                self.alive[i] = False
            out.append(t)
        return out

    def close(self):
        assert not self.closed
        self.closed = True
        self.b.open_runs -= 1


class ScriptedBackend:
    def __init__(self, max_batch=3, capacity=64 * 8):
        self.max_batch, self.capacity = max_batch, capacity
        self.batches, self.steps, self.open_runs = [], 0, 0
        self.streams = []

    def token_capacity(self):
        return self.capacity

    def tokens_needed(self, prompt_len, max_new):
        return -(-(prompt_len + max_new) // 64) * 64

    def start(self, prompts, max_new, sampling, stop_ids, streams):
        assert self.open_runs == 0, "a batch started before the previous one was closed"
        self.open_runs += 1
        self.batches.append([len(p) for p in prompts])
        self.streams.append(list(streams))
        self.sampling = sampling
        return ScriptedRun(self, prompts, max_new, stop_ids)


def test_requests_are_served_in_batches_one_after_another():
    be = ScriptedBackend(max_batch=3)
    loop = GenerationLoop(be)
    prompts = [[10 * i] * (i + 1) for i in range(7)]
    out = loop.run(prompts, 4)
    assert be.batches == [[1, 2, 3], [4, 5, 6], [7]] and be.open_runs == 0
    assert be.streams == [[0, 1, 2], [3, 4, 5], [6]]        # a request's stream is its index
    assert out == [[10 * i + 1 + j for j in range(4)] for i in range(7)]


def test_batches_also_close_on_cache_room():
    be = ScriptedBackend(max_batch=8, capacity=64 * 4)
    loop = GenerationLoop(be)
    prompts = [[1] * 100, [2] * 20, [3] * 60, [4] * 5]      # need 128, 64, 128, 64 tokens of room
    loop.run(prompts, 10)
    assert be.batches == [[100, 20], [60, 5]]
    with pytest.raises(GenerationError, match="needs room for 320"):
        loop.run([[1] * 300], 10)


def test_stop_tokens_end_a_sequence_and_the_batch_ends_with_its_last():
    be = ScriptedBackend(max_batch=4)
    loop = GenerationLoop(be)
    out = loop.run([[5], [50], [500]], [6, 3, 6], stop_token_ids=[8, 503])
    assert out == [[6, 7, 8], [51, 52, 53], [501, 502, 503]]    # stop token kept, nothing after
    assert be.steps == 3                                        # no step after the last one ended
    be2 = ScriptedBackend(max_batch=4)
    steps = list(GenerationLoop(be2).stream([[5], [50]], 5, stop_token_ids=[7]))
    assert steps == [[6, 51], [7, 52], [-1, 53], [-1, 54], [-1, 55]] and be2.open_runs == 0


def test_per_request_budgets_and_zero_budget():
    be = ScriptedBackend()
    out = GenerationLoop(be).run([[1], [2], [3]], [2, 0, 1])
    assert out == [[2, 3], [], [4]] and be.batches == [[1, 1]]


def test_stream_is_one_batch_only_and_inputs_are_checked():
    be = ScriptedBackend(max_batch=2)
    loop = GenerationLoop(be)
    with pytest.raises(GenerationError, match="do not fit one batch"):
        list(loop.stream([[1], [2], [3]], 2))
    with pytest.raises(GenerationError, match="empty"):
        loop.run([[1], []], 2)
    with pytest.raises(GenerationError, match="one per prompt"):
        loop.run([[1], [2]], [1])
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)


def test_a_batch_is_closed_when_its_consumer_stops_early_or_fails():
    be = ScriptedBackend()
    gen = GenerationLoop(be).stream([[1], [2]], 10)
    next(gen)
    gen.close()
    assert be.open_runs == 0

    class Broken(ScriptedRun):
        def next_tokens(self):
            raise RuntimeError("device lost")
    be2 = ScriptedBackend()
    be2.start = lambda *a: (setattr(be2, "open_runs", 1), Broken(be2, a[0], a[1], a[3]))[1]
    with pytest.raises(RuntimeError, match="device lost"):
        GenerationLoop(be2).run([[1]], 3)
    assert be2.open_runs == 0


def test_rows_accept_lists_tuples_arrays_and_tensors():
    import numpy as np
    import torch
    assert as_rows([[1, 2], (3,)]) == [[1, 2], [3]]
    assert as_rows(np.array([[1, 2], [3, 4]])) == [[1, 2], [3, 4]]
    assert as_rows(torch.tensor([[5, 6]])) == [[5, 6]]
    assert as_rows([torch.tensor([7]), np.array([8, 9])]) == [[7], [8, 9]]
