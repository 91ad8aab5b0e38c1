"""bin/trace_run as a user drives it: steps on standard input, logits in files."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain
from tests.plain import tiny_models

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(folder, dtype, out, steps, max_tokens):
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", str(folder), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(max_tokens)],
                          input="".join(json.dumps(s) + "\n" for s in steps), text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    return proc


def read(out, step, vocab):
    a = np.fromfile(os.path.join(str(out), f"{step}.f32"), dtype="<f4")
    return torch.from_numpy(a.reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_whole_tail_and_unequal_batches(tmp_path, dtype):
    cfg = tiny_models.TINY_B
    vocab = cfg["vocab_size"]
    folder = helpers.make_folder(tmp_path / "model", cfg, 1)
    model = helpers.plain_model(folder)
    seqs = tiny_models.random_prompts(cfg, [70, 33, 5, 129], seed=3)
    want = [plain.logits(model, s) for s in seqs]
    steps, expect = [], {}
    n = 0
    # (1) each request alone and whole
    for i, s in enumerate(seqs):
        steps.append({"step": n, "entries": [{"id": f"w{i}", "tokens": s, "want": list(range(len(s)))}],
                      "end": [f"w{i}"]})
        expect[n] = want[i]
        n += 1
    # (2) request 0: head whole, last 32 one by one; only some places wanted in the head
    s = seqs[0]
    head = len(s) - 32
    steps.append({"step": n, "entries": [{"id": "t", "tokens": s[:head], "want": [0, head - 1]}], "end": []})
    expect[n] = want[0][[0, head - 1]]
    n += 1
    for j in range(head, len(s)):
        steps.append({"step": n, "entries": [{"id": "t", "tokens": [s[j]], "want": [0]}],
                      "end": ["t"] if j == len(s) - 1 else []})
        expect[n] = want[0][j:j + 1]
        n += 1
    # (3) two batches of unequal lengths, one after the other; shorter requests end earlier;
    # a step in which nothing is wanted writes no file
    for rnd, (members, heads) in enumerate((([1, 2, 3], [30, 2, 100]), ([0, 2], [64, 5]))):
        ids = {i: f"b{rnd}_{i}" for i in members}
        steps.append({"step": n, "entries": [{"id": ids[i], "tokens": seqs[i][:h], "want": [h - 1]}
                                            for i, h in zip(members, heads)],
                      "end": [ids[i] for i, h in zip(members, heads) if h == len(seqs[i])]})
        expect[n] = torch.stack([want[i][h - 1] for i, h in zip(members, heads)])
        n += 1
        done = dict(zip(members, heads))
        while any(done[i] < len(seqs[i]) for i in members):
            live = [i for i in members if done[i] < len(seqs[i])]
            wanted = n % 3 != 0
            steps.append({"step": n, "entries": [{"id": ids[i], "tokens": [seqs[i][done[i]]],
                                                 "want": [0] if wanted else []} for i in live],
                          "end": [ids[i] for i in live if done[i] + 1 == len(seqs[i])]})
            if wanted:
                expect[n] = torch.stack([want[i][done[i]] for i in live])
            for i in live:
                done[i] += 1
            n += 1
    # the most live tokens at once, each request rounded up to 64: the batch of three
    max_tokens = 64 + 64 + 192
    replay(folder, dtype, tmp_path / "out", steps, max_tokens)
    files = sorted(os.listdir(tmp_path / "out"))
    assert files == sorted(f"{k}.f32" for k in expect)
    for k, w in expect.items():
        got = read(tmp_path / "out", k, vocab)
        assert got.shape == w.shape
        err = (got - w).abs().max().item() / want[0].abs().max().item()
        assert err <= helpers.TOL[dtype], f"step {k}: {err:.3e}"


def test_replay_errors_are_loud(tmp_path):
    cfg = tiny_models.TINY_A
    folder = helpers.make_folder(tmp_path / "model", cfg, 0)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": []}], "end": []}]
    proc = subprocess.run([sys.executable, TRACE_RUN, "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input=json.dumps(steps[0]) + "\n", text=True, capture_output=True, timeout=600)
    assert proc.returncode != 0 and ("cache is full" in proc.stderr or "limit" in proc.stderr)
