"""What bench.py promises without a GPU: more than one GPU is refused with exit code 2, the reference arm
prints one line of JSON (here, without a GPU, why it cannot be timed), and the sizes of every shape are
the ones BASELINE.json names."""

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


def test_reference_arm_prints_one_json_line_and_never_fails():
    """With a GPU and a copy of the reference under baseline/_ref it times the reference's own
    Engine.generate; without either it says which one is missing."""
    p = run("--impl", "reference")
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference"
    import torch
    if not torch.cuda.is_available() or not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "engine")):
        assert isinstance(rec["unavailable"], str) and rec["unavailable"]
        assert "GPU" in rec["unavailable"] or "CUDA" in rec["unavailable"] or "baseline/_ref" in rec["unavailable"]


def test_every_shape_follows_the_baseline_file():
    sys.path.insert(0, ROOT)
    import bench
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        configs = json.load(f)["configs"]
    for shape, (index, preset, work) in bench.SHAPES.items():
        cfg = bench.shape_config(shape)
        for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "intermediate_size", "vocab_size"):
            assert f"{key}={cfg[key]}" in configs[index], (shape, key)
            assert cfg[key] == preset[key], (shape, key)
        assert f"tie_word_embeddings={'true' if cfg['tie_word_embeddings'] else 'false'}" in configs[index]
    lengths = [len(p) for p in bench.make_prompts("8b", 16, 1000)]
    assert len(lengths) == 16 and min(lengths) >= 64 and max(lengths) <= 2048 and len(set(lengths)) > 8
    assert lengths == [len(p) for p in bench.make_prompts("8b", 16, 1000)]          # seeded


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
