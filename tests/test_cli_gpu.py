"""The command line as a user runs it: ``random-model`` writes a folder, ``generate`` loads it and
prints token ids, and in 32-bit they are the plain implementation's greedy tokens."""

import json
import os
import subprocess
import sys

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.plain import tiny_models

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(*args):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-m", "enginekernel_b200", *args], capture_output=True, text=True,
                       cwd=ROOT, env=env, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout


def test_random_model_then_generate(tmp_path):
    cfg = dict(tiny_models.TINY_B)
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    out = run_cli("random-model", "--config", str(config_file), "--seed", "11", "--out", str(folder))
    assert str(folder) in out
    assert (folder / "config.json").exists() and (folder / "model.safetensors").exists()

    prompts = tiny_models.random_prompts(cfg, (3, 40, 17), seed=4)
    ids = ";".join(",".join(str(t) for t in p) for p in prompts)
    out = run_cli("generate", "--model", str(folder), "--dtype", "float32", "--prompt-ids", ids,
                  "--out-len", "9")
    rows = [json.loads(line) for line in out.strip().splitlines()]
    assert [r["request"] for r in rows] == [0, 1, 2]
    model = plain.PlainModel(str(folder), torch.float32)
    want = [plain.greedy(model, p, 9) for p in prompts]
    assert [r["tokens"] for r in rows] == want
    assert max(len(set(w)) for w in want) >= 4          # not one repeated token

    # a stop token ends its request; the others go on
    stop = want[1][3]
    out = run_cli("generate", "--model", str(folder), "--dtype", "float32", "--prompt-ids", ids,
                  "--out-len", "9", "--stop-ids", str(stop))
    rows = [json.loads(line) for line in out.strip().splitlines()]
    for r, w in zip(rows, want):
        cut = w.index(stop) + 1 if stop in w else len(w)
        assert r["tokens"] == w[:cut]
