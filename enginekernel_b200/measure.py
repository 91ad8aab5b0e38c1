"""Where a step's time goes: each kernel of a step timed on its own, against its roofline.

One step is run eagerly under a :class:`~enginekernel_b200.ops.lib.LaunchRecord`, which keeps
every launch (entry point, arguments, and what the launcher says the launch has to move and
compute).  Then, for each entry point, the launches of that entry point alone are issued again
into a CUDA graph - the q/k/v product of every layer one after the other, each with its own
weights - and replays of that graph are timed with CUDA events, with the L2 overwritten before
each replay.  A kernel's time divided into its bytes (or flops) is its achieved rate; over the
measured peak that is its fraction of the roofline.  The sum over the entry points against the
whole captured step shows what the boundaries between kernels cost (or hide).

The reference times its kernels the same way - a callable captured in a graph, replays timed,
weights cycled over all layers so that the L2 does not help, a table from kernel to bytes and
"% of HBM peak" (bench/profile2.py:12-27, 42-44, 62-70; bench/ablate.py:13-28).
"""

from __future__ import annotations

import statistics
from typing import Callable, Dict, List, Optional

import torch

from .ops.lib import LaunchRecord

L2_FLUSH_BYTES = 256 << 20        # twice the 126 MB L2


def record_launches(run_step: Callable[[], None]) -> LaunchRecord:
    """Run ``run_step`` (which issues one step's kernels on the current stream) on a side
    stream and return the record of its launches."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with LaunchRecord() as rec:
            run_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return rec


class _Flusher:
    def __init__(self, device):
        self.buf = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=device)

    def __call__(self):
        self.buf.zero_()
        # keep the device busy while the host queues the timed work, so that no host gap is timed
        torch.cuda._sleep(200_000)


@torch.inference_mode()
def time_record(record: LaunchRecord, name: Optional[str], iters: int, flush: _Flusher) -> float:
    """Median milliseconds of one replay of the recorded launches of ``name`` (all, if None)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        record.issue(side.cuda_stream, name)            # warm: modules loaded, library workspaces
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        record.issue(torch.cuda.current_stream().cuda_stream, name)
    times = []
    for _ in range(iters):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    del graph
    return statistics.median(times)


def kernel_table(record: LaunchRecord, peaks: Dict[str, float], iters: int = 7,
                 between: Optional[Callable[[], None]] = None) -> List[dict]:
    """One row per entry point of ``record``: launches, microseconds of all of them together,
    bytes, flops, and the fraction of the bound that is nearer (``peaks``: ``hbm_gbs``,
    ``bf16_tflops``).  ``between`` is called after each entry point was timed (to put back state
    that its launches advance)."""
    device = torch.cuda.current_device()
    flush = _Flusher(device)
    rows = []
    for name in record.names():
        ms = time_record(record, name, iters, flush)
        if between is not None:
            between()
        cost = record.cost(name)
        row = {"kernel": name, "launches": cost["launches"], "us": round(ms * 1e3, 2)}
        seconds = ms / 1e3
        t_mem = cost["bytes"] / (peaks["hbm_gbs"] * 1e9)
        t_math = cost["flops"] / (peaks["bf16_tflops"] * 1e12)
        if cost["bytes"]:
            row["gb"] = round(cost["bytes"] / 1e9, 4)
        if cost["flops"]:
            row["gflop"] = round(cost["flops"] / 1e9, 2)
        if cost["bytes"] or cost["flops"]:
            if t_math > t_mem:
                row["bound"], row["frac"] = "tensor", round(t_math / seconds, 3)
            else:
                row["bound"], row["frac"] = "hbm", round(t_mem / seconds, 3)
        rows.append(row)
    return rows


def decode_step_table(state, peaks: Dict[str, float], iters: int = 7) -> dict:
    """Per-kernel table of one decode step of ``state`` (a
    :class:`~enginekernel_b200.engine.decode.DecodeState` of a running batch).  The step that is
    recorded is a real one (every sequence moves on by a token); the state that the timed
    replays advance is put back afterwards."""
    rec = record_launches(state._body)
    saved = state.snapshot()
    rows = kernel_table(rec, peaks, iters, between=lambda: state.restore(saved))
    flush = _Flusher(torch.cuda.current_device())
    whole = time_record(rec, None, iters, flush)
    state.restore(saved)
    torch.cuda.synchronize()
    return {"kernels": rows, "sum_us": round(sum(r["us"] for r in rows), 1),
            "step_us": round(whole * 1e3, 1)}


def prefill_step_table(run_step: Callable[[], None], peaks: Dict[str, float], iters: int = 5) -> dict:
    """Per-kernel table of a prompt step; ``run_step`` runs it once (the cache rows it writes
    are written again, with the same values, by the timed replays)."""
    rec = record_launches(run_step)
    rows = kernel_table(rec, peaks, iters)
    return {"kernels": rows, "sum_us": round(sum(r["us"] for r in rows), 1)}
