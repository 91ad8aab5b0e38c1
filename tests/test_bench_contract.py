"""What bench.py promises without a GPU: more than one GPU is refused with exit code 2, the reference arm
says why it is unavailable, and the default sizes are the ones BASELINE.json names."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True,
                          text=True, cwd=ROOT, timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
    p = run("--gpus", "2")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1


def test_reference_arm_is_unavailable_and_says_why():
    p = run("--impl", "reference")
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and rec["unavailable"]


def test_default_sizes_are_the_ones_the_baseline_names():
    sys.path.insert(0, ROOT)
    import bench
    cfg = bench.benchmark_config()
    assert cfg["architectures"] == ["Qwen3ForCausalLM"]
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        text = json.load(f)["configs"][2]
    for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                "intermediate_size", "vocab_size"):
        assert f"{key}={cfg[key]}" in text, key
