"""Decode and prefill throughput of the Qwen3-4B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences that each hold a 2,048-token prompt
(context limit 4,096).  ``value`` is decoded tokens per second over K captured-graph
replays timed with CUDA events; ``e2e`` is the same through ``Engine.generate`` with
prompts given as host lists and every step's tokens read back on the host; ``prefill``
is one 2,048-token prompt; ``roofline`` divides the bytes a decode step has to read
(each weight once plus the live cache) by its time; ``points`` are batch 1 and 64.
The reference's own local benchmark (bench/bench.py:18-22, 61-75) times whole
``generate`` calls on a real checkpoint; it publishes no numbers.  One line of JSON is
printed.  The inputs of a step (8 GB of weights) are larger than the L2.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PRESET_4B = {   # BASELINE.json configs[2]; re-read from the file when it is there
    "num_hidden_layers": 36, "hidden_size": 2560, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728, "vocab_size": 151936,
    "rope_theta": 5000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
}
PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def benchmark_config():
    cfg = dict(PRESET_4B)
    path = os.path.join(ROOT, "BASELINE.json")
    try:
        with open(path) as f:
            text = json.load(f)["configs"][2]
        for key, cast in (("num_hidden_layers", int), ("hidden_size", int),
                          ("num_attention_heads", int), ("num_key_value_heads", int),
                          ("head_dim", int), ("intermediate_size", int), ("vocab_size", int),
                          ("rope_theta", float), ("rms_norm_eps", float)):
            m = re.search(key + r"=([0-9.e+-]+)", text)
            if m:
                cfg[key] = cast(float(m.group(1)))
        m = re.search(r"tie_word_embeddings=(true|false)", text)
        if m:
            cfg["tie_word_embeddings"] = m.group(1) == "true"
    except (OSError, KeyError, IndexError, ValueError):
        pass
    cfg["architectures"] = ["Qwen3ForCausalLM"]
    return cfg


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
               "source": "measured"}
        if "bf16_tflops_sustained" in raw:
            out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
        return out
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is not installable offline: pip reports neither setup.py "
                          "nor pyproject.toml in it, and its kernels are Triton code tuned for sm_90"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this library runs on a single B200); --gpus {args.gpus} is not run")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from enginekernel_b200 import Engine
    from enginekernel_b200.config import Qwen3Config
    from enginekernel_b200.ops.lib import loaded_libraries

    raw = benchmark_config()
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(raw)
    pk = peaks()
    torch.manual_seed(0)
    biggest = max(args.batch, 1 if args.skip_points else 64)
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=biggest * CONTEXT,
                                max_batch=biggest, max_len=CONTEXT)
    g = torch.Generator().manual_seed(0)

    def prompts(b):
        return torch.randint(0, cfg.vocab_size, (b, PROMPT_LEN), generator=g).tolist()

    # ---- prefill of 2,048 tokens -------------------------------------------------------
    one = prompts(1)[0]
    times = []
    for it in range(4 + 5):                      # 4 warm-ups (clocks, workspace), median of 5
        slot = engine.open_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([(slot, one, [PROMPT_LEN - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.close_sequence(slot)
        if it >= 4:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)
    L, H, NH, NKV, D, I, V = (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads,
                              cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size,
                              cfg.vocab_size)
    per_token_linear = 2 * L * (H * (NH + 2 * NKV) * D + NH * D * H + 3 * H * I)
    attn_flops = L * 4 * NH * D * PROMPT_LEN * (PROMPT_LEN + 1) / 2
    prefill_flops = per_token_linear * PROMPT_LEN + attn_flops + 2 * H * V
    prefill = {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode --------------------------------------------------------------------------
    def decode(b, steps, sample_clocks=False):
        run = engine.backend.start(prompts(b), [warmup + steps + 4] * b, engine_sampling(), [],
                                   list(range(b)))
        try:
            st = run.state
            for _ in range(warmup):
                st.step()
            torch.cuda.synchronize()
            sampler = ClockSampler() if sample_clocks else None
            if sampler:
                sampler.start()
                time.sleep(0.3)
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                st.step()
            e.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(e) / steps
            clocks = sampler.stop() if sampler else None
            return ms, clocks, st.launches_per_step
        finally:
            run.close()

    def engine_sampling():
        from enginekernel_b200 import SamplingParams
        return SamplingParams()

    ms_step, clocks, launches = decode(args.batch, args.steps, sample_clocks=True)
    value = args.batch / (ms_step / 1e3)
    weight_bytes = engine.model.weight_bytes_read_per_step()
    kv_per_token = 2 * L * NKV * D * 2
    mean_context = PROMPT_LEN + warmup + args.steps / 2
    step_bytes = weight_bytes + args.batch * mean_context * kv_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms_b, _, _ = decode(b, max(16, args.steps // 2))
            points[f"decode_b{b}"] = b / (ms_b / 1e3)

    # ---- end to end through Engine.generate --------------------------------------------
    host_prompts = prompts(args.batch)
    list(engine.generate(host_prompts, 4))                           # warm the shape
    n_new = args.steps + 1
    t_first = None
    count = 0
    for toks in engine.generate(host_prompts, n_new):
        if t_first is None:
            t_first = time.perf_counter()
        else:
            count += 1
    t_last = time.perf_counter()
    e2e_value = args.batch * count / (t_last - t_first)
    plan_bytes = 4 * (4 * args.batch * PROMPT_LEN + args.batch + 1)   # ids, positions, slots, rows
    e2e = {"value": e2e_value, "unit": "tok/s",
           "h2d_bytes_per_step": plan_bytes / max(count, 1), "d2h_bytes_per_step": 4 * args.batch}

    out = {
        "metric": "decode tok/s (Qwen3-4B shape, batch 8, 2,048-token prompts)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {
            "model": "Qwen3-4B shape (Qwen3ForCausalLM)", "num_hidden_layers": full_layers,
            "layers_run": cfg.num_hidden_layers, "hidden_size": H, "num_attention_heads": NH,
            "num_key_value_heads": NKV, "head_dim": D, "intermediate_size": I, "vocab_size": V,
            "tie_word_embeddings": cfg.tie_word_embeddings, "rope_theta": cfg.rope_theta,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "parallelism": "none (1 GPU)", "l2": "step inputs (8 GB of weights) exceed the 126 MB L2",
            "peaks": pk["source"]},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches * args.steps,
        "prefill": prefill, "roofline": roofline, "points": points,
        "kernel_libraries": sorted(os.path.basename(p) for p in loaded_libraries().values()),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
