"""Shared helpers of the GPU tests: model folders, and ways of cutting requests into steps."""

from __future__ import annotations

import torch

from tests.plain import qwen3_plain as plain
from tests.plain import tiny_models

# Limits on |engine - plain| / max|plain| for logits.  32-bit: summation-order noise only.
# bfloat16: the engine rounds activations to 8 mantissa bits at each matrix product while
# the plain implementation runs in 32-bit on the same bfloat16-rounded weights; 2e-2 of the
# tensor's scale is the reference's own bound for its bfloat16 kernels
# (bench/test_kernels.py:18-33) and is used unchanged here for whole-model logits.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def rel_err(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


def make_folder(path, cfg, seed, **kw):
    return tiny_models.write_tiny(str(path), cfg, seed, dtype=torch.bfloat16, **kw)


def whole(engine, tokens):
    """One request alone, all tokens in one step, logits everywhere."""
    slot = engine.open_sequence()
    try:
        return engine.step([(slot, tokens, list(range(len(tokens))))]).cpu()
    finally:
        engine.close_sequence(slot)


def tail_one_by_one(engine, tokens, tail=32):
    """The head in one step, then the last ``tail`` tokens one per step."""
    head = max(1, len(tokens) - tail)
    slot = engine.open_sequence()
    try:
        rows = [engine.step([(slot, tokens[:head], list(range(head)))]).cpu()]
        for t in tokens[head:]:
            rows.append(engine.step([(slot, [t], [0])]).cpu())
        return torch.cat(rows, 0)
    finally:
        engine.close_sequence(slot)


def batch_then_steps(engine, seqs, heads):
    """Requests that start together: their heads (unequal lengths) in one step, then one
    token each per step; a request that runs out of tokens ends and gives its slot back
    while the others go on.  Returns the logits of every request at every position."""
    slots = [engine.open_sequence() for _ in seqs]
    out = [[] for _ in seqs]
    live = list(range(len(seqs)))
    try:
        logits = engine.step([(slots[i], seqs[i][:heads[i]], list(range(heads[i]))) for i in live]).cpu()
        r = 0
        for i in live:
            out[i].append(logits[r:r + heads[i]])
            r += heads[i]
        done = list(heads)
        while True:
            for i in list(live):
                if done[i] >= len(seqs[i]):
                    engine.close_sequence(slots[i])
                    slots[i] = None
                    live.remove(i)
            if not live:
                break
            logits = engine.step([(slots[i], [seqs[i][done[i]]], [0]) for i in live]).cpu()
            for r, i in enumerate(live):
                out[i].append(logits[r:r + 1])
                done[i] += 1
    finally:
        for s in slots:
            if s is not None:
                engine.close_sequence(s)
    return [torch.cat(o, 0) for o in out]


def plain_model(folder):
    return plain.PlainModel(str(folder), torch.float32)


def make_context(dtype, device, positions, slots, cu_seqlens, max_context=None):
    """A StepContext over explicit per-token positions and slots (for tests of parts alone)."""
    from enginekernel_b200.parts.base import StepContext, Workspace
    i32 = dict(dtype=torch.int32, device=device)
    n = len(positions)
    lens = [b - a for a, b in zip(cu_seqlens[:-1], cu_seqlens[1:])]
    return StepContext(
        n_tokens=n, n_seqs=len(lens), token_ids=torch.zeros(n, **i32),
        positions=torch.tensor(positions, **i32), token_slot=torch.tensor(slots, **i32),
        cu_seqlens=torch.tensor(cu_seqlens, **i32), is_decode=all(x == 1 for x in lens),
        max_new=max(lens), max_context=max_context or (max(positions) + 1), dtype=dtype,
        device=torch.device(device), workspace=Workspace(device), host_positions=list(positions),
        host_token_slot=list(slots), host_cu_seqlens=list(cu_seqlens))
