"""Batches on the device: one prefill step, then decode steps that need no host.

A batch's decode state lives in device tensors (one row per sequence): the token to
feed next, its position, the sequence's slot, how many draws it has made, how many
tokens it may still emit.  One decode step is the model's forward for one token per
sequence, the sampling kernel and a state-advance kernel; the whole step is captured in a
CUDA graph per (batch size, context bucket) and replayed, a few replays ahead of the token
the host is reading (tokens come back through pinned memory and events).  This follows the
reference (engine/engine.py:284-330 capture, 604-634 replay loop with LOOKAHEAD), with
per-sequence positions and stop conditions instead of one shared length and a fixed step
count.
"""

from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..cache.pages import PAGE
from ..ops import kernels
from ..parts.base import StepContext, Workspace
from ..sampling.params import SamplingParams
from .runner import ModelRunner, StepEntry

LOOKAHEAD = 2
CONTEXT_BUCKET = 1024


class DecodeState:
    """Device state of a batch of ``batch`` sequences, and the captured step."""

    def __init__(self, runner: ModelRunner, batch: int, bucket: int, max_steps: int, use_graph: bool):
        dev = runner.device
        self.runner, self.batch, self.bucket, self.max_steps = runner, batch, bucket, max_steps
        i32 = dict(dtype=torch.int32, device=dev)
        self.token_ids = torch.zeros(batch, **i32)
        self.positions = torch.full((batch,), -1, **i32)
        self.token_slot = torch.zeros(batch, **i32)
        self.draws = torch.zeros(batch, **i32)
        self.remaining = torch.zeros(batch, **i32)
        self.streams = torch.zeros(batch, **i32)
        self.sampled = torch.zeros(batch, **i32)
        self.rows = torch.arange(batch, **i32)
        self.cu_seqlens = torch.arange(batch + 1, **i32)
        self.out_tokens = torch.zeros((max_steps, batch), **i32)
        self.step_index = torch.zeros(1, **i32)
        self.stop_ids = torch.zeros(64, **i32)
        self.n_stop = 0
        self.settings = kernels.sampling_settings(0.0, 0, 0, dev)
        self.top_k = 0                           # host copy: chooses the sampling kernel
        self.part_score = torch.zeros(batch * kernels.SAMPLE_SEGMENTS, dtype=torch.float32, device=dev)
        self.part_index = torch.zeros(batch * kernels.SAMPLE_SEGMENTS, **i32)
        self.workspace = Workspace(dev)          # owned by the graph: never regrown elsewhere
        self.graph = None
        self.use_graph = use_graph
        self.launches_per_step = 0               # kernel launcher calls in one step
        self.ctx = StepContext(
            n_tokens=batch, n_seqs=batch, token_ids=self.token_ids, positions=self.positions,
            token_slot=self.token_slot, cu_seqlens=self.cu_seqlens, is_decode=True, max_new=1,
            max_context=bucket, dtype=runner.model.dtype, device=dev, workspace=self.workspace)

    def configure(self, stop_ids: Sequence[int], sampling: SamplingParams):
        if len(stop_ids) > self.stop_ids.numel():
            raise ValueError(f"at most {self.stop_ids.numel()} stop tokens")
        # the stop count and the choice of sampling kernel are fixed in a captured step
        if (self.n_stop != len(stop_ids) or (self.top_k > 0) != (sampling.top_k > 0)) \
                and self.graph is not None:
            self.graph = None
        self.n_stop = len(stop_ids)
        self.top_k = sampling.top_k
        if stop_ids:
            self.stop_ids[:len(stop_ids)] = torch.tensor(list(stop_ids), dtype=torch.int32)
        self.settings.copy_(kernels.sampling_settings(sampling.temperature, sampling.top_k,
                                                      sampling.seed, self.settings.device))

    def sample_and_advance(self, logits):
        if logits.shape[-1] < 4096:
            kernels.sample(self.sampled, logits, 0.0, 0, 0, streams=self.streams, draws=self.draws,
                           active=self.positions, n_rows=self.batch, dyn=self.settings)
        elif self.top_k > 0:
            kernels.sample_cluster(self.sampled, logits, 0.0, 0, 0, streams=self.streams,
                                   draws=self.draws, active=self.positions, n_rows=self.batch,
                                   dyn=self.settings)
        else:
            kernels.sample_wide(self.sampled, logits, 0.0, 0, self.part_score, self.part_index,
                                streams=self.streams, draws=self.draws, active=self.positions,
                                n_rows=self.batch, dyn=self.settings)
        kernels.decode_advance(self.sampled, self.token_ids, self.positions, self.draws,
                               self.remaining, self.out_tokens, self.step_index, self.stop_ids,
                               self.n_stop, self.batch)

    _ADVANCED = ("token_ids", "positions", "draws", "remaining", "sampled", "step_index")

    def snapshot(self):
        """Copies of the arrays a step advances (for measurements that replay steps and then put
        the batch back where it was)."""
        return {name: getattr(self, name).clone() for name in self._ADVANCED}

    def restore(self, saved) -> None:
        for name, value in saved.items():
            getattr(self, name).copy_(value)

    def _body(self):
        model, cache = self.runner.model, self.runner.cache
        logits = model.forward(self.ctx, cache, self.rows, self.batch)
        self.sample_and_advance(logits)

    def step(self):
        """Enqueue one decode step."""
        if not self.use_graph:
            self._body()
            return
        if self.graph is None:
            self._capture()
        self.graph.replay()

    def _capture(self):
        # Warm up with every row switched off: kernels are loaded and buffers sized, the
        # cache and the state stay as they are.
        saved = (self.positions.clone(), self.step_index.clone())
        self.positions.fill_(-1)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..ops.lib import launch_calls
        g = torch.cuda.CUDAGraph()
        before = launch_calls()
        with torch.cuda.graph(g):
            self._body()
        self.launches_per_step = launch_calls() - before
        self.positions.copy_(saved[0])
        self.step_index.copy_(saved[1])
        torch.cuda.synchronize()
        self.graph = g


class DeviceBatchRun:
    """One batch in flight (see :mod:`enginekernel_b200.engine.generate` for the interface)."""

    def __init__(self, backend: "DeviceBackend", prompts, max_new, sampling: SamplingParams,
                 stop_ids, streams):
        self.backend = backend
        runner, cache = backend.runner, backend.runner.cache
        self.batch = len(prompts)
        self.slots: List[int] = []
        self.closed = False
        try:
            for p, n in zip(prompts, max_new):
                s = cache.open()
                self.slots.append(s)
                cache.reserve(s, len(p) + n)
            total = max(len(p) + n for p, n in zip(prompts, max_new))
            self.max_steps = max(max_new)
            st = backend.state_for(self.batch, total, self.max_steps)
            self.state = st
            st.configure(stop_ids, sampling)
            # prefill: every prompt in one step, logits at each prompt's last token
            logits = runner.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(self.slots, prompts)])
            i32 = dict(dtype=torch.int32)
            st.token_slot.copy_(torch.tensor(self.slots, **i32))
            st.streams.copy_(torch.tensor([int(x) & 0x7FFFFFFF for x in streams], **i32))
            st.positions.copy_(torch.tensor([len(p) - 1 for p in prompts], **i32))
            st.remaining.copy_(torch.tensor(list(max_new), **i32))
            st.draws.zero_()
            st.step_index.zero_()
            st.sample_and_advance(logits)          # the first token is draw 0, step 0
        except Exception:
            self.close()
            raise
        self.launched = 1                          # steps whose tokens are (being) computed
        self.read = 0
        self.host = backend.host_tokens(self.max_steps, self.batch)
        self.events = [torch.cuda.Event() for _ in range(LOOKAHEAD + 2)]
        self._fetch(0)

    def _fetch(self, step: int):
        self.host[step, :self.batch].copy_(self.state.out_tokens[step], non_blocking=True)
        self.events[step % len(self.events)].record()

    def _launch(self):
        self.state.step()
        self._fetch(self.launched)
        self.launched += 1

    def next_tokens(self) -> List[int]:
        if self.read >= self.max_steps:
            raise RuntimeError("the batch has no more steps")
        # The first token is handed over before the decode queue is filled (as the reference does,
        # engine/engine.py:625-627): nothing stands between the prompt and its first token, not
        # even a graph capture.  After that the device is kept ahead of the reader, never past the
        # last step any row can need.
        if self.read > 0:
            self._fill()
        self.events[self.read % len(self.events)].synchronize()
        toks = self.host[self.read, :self.batch].tolist()
        self.read += 1
        return toks

    def _fill(self):
        while self.launched < min(self.read + 1 + LOOKAHEAD, self.max_steps):
            self._launch()

    def close(self):
        if self.closed:
            return
        self.closed = True
        if self.slots:
            torch.cuda.current_stream().synchronize()   # queued steps still write these pages
        cache = self.backend.runner.cache
        for s in self.slots:
            cache.close(s)
        self.slots = []
        self.backend.runner.check_kernels()


class DeviceBackend:
    def __init__(self, runner: ModelRunner, max_batch: int, use_graph: bool = True):
        self.runner = runner
        self.max_batch = max(1, min(max_batch, runner.cache.num_slots, 1024))
        self.use_graph = use_graph
        self._states: Dict[tuple, DecodeState] = {}
        self._host = None

    def token_capacity(self) -> int:
        return self.runner.cache.free_tokens()

    def tokens_needed(self, prompt_len: int, max_new: int) -> int:
        return -(-(prompt_len + max_new) // PAGE) * PAGE

    def state_for(self, batch: int, total_len: int, max_steps: int) -> DecodeState:
        bucket = -(-total_len // CONTEXT_BUCKET) * CONTEXT_BUCKET
        key = (batch, bucket)
        st = self._states.get(key)
        if st is None or st.max_steps < max_steps:
            if len(self._states) >= 8:                 # graphs hold memory: keep a few
                self._states.pop(next(iter(self._states)))
            st = DecodeState(self.runner, batch, bucket, max(max_steps, 256), self.use_graph)
            self._states[key] = st
        return st

    def host_tokens(self, steps: int, batch: int):
        h = self._host
        if h is None or h.shape[0] < steps or h.shape[1] < batch:
            h = torch.zeros((max(steps, 256), max(batch, 8)), dtype=torch.int32, pin_memory=True)
            self._host = h
        return h

    def start(self, prompts, max_new, sampling, stop_ids, streams) -> DeviceBatchRun:
        return DeviceBatchRun(self, prompts, max_new, sampling, stop_ids, streams)
