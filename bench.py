"""Decode and prefill throughput of Qwen3 shapes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 4b|8b|0.6b] [--impl ours|reference]
                    [--batch B] [--layers L] [--skip-points] [--skip-kernels]

The shapes and workloads are the ones BASELINE.json names (its configs[2], [3], [4]):

4b    (default) batch 8, 2,048-token prompts, context limit 4,096; decode at batch 1 and 64 and a
      prefill of 2,048 tokens beside it
8b    a ragged batch of 16 prompts with seeded lengths U[64, 2048], then 256 decode steps, untied head
0.6b  batch 64 with caches of 8,192 tokens

A step is one decode step of the batch.  ``value`` is decoded tokens per second over K replays of
the captured step timed with CUDA events, repeated until at least a second of device time has
been timed (``repeats``).  ``e2e`` times whole ``Engine.generate`` calls the way the reference's
own harness does (bench/bench.py:30-38, 61-75): host token lists in, the prompt step and every
decode step inside the clock, every step's tokens read back on the host; it gives tokens per
second of the whole call, the time to the first token, and the rate after the first token.
``prefill`` is one 2,048-token prompt; ``roofline`` divides the bytes a decode step has to read
(each weight once plus the live cache) by its time; ``kernels`` times each kernel of the decode
step and of the prompt step on its own (:mod:`enginekernel_b200.measure`) against the measured
peaks.  One line of JSON is printed.  The inputs of a step (gigabytes of weights) are larger than
the L2.

``--impl reference`` runs the unmodified reference from ``baseline/_ref`` (a plain copy of its
tree) on the same workload: its stock ``Engine(model_path).generate(input_ids, max_new_tokens)``
(engine/engine.py:770-830) on a folder of random weights of the same shape, with none of this
repository's kernels, models or engine on that path.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# What BASELINE.json's configs say, kept here for runs without that file; re-read from it when it
# is there.  (index in "configs", sizes, workload)
SHAPES = {
    "4b": (2, {"num_hidden_layers": 36, "hidden_size": 2560, "num_attention_heads": 32,
               "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
               "vocab_size": 151936, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6,
               "tie_word_embeddings": True, "max_position_embeddings": 4096},
           {"batch": 8, "prompt": 2048, "context": 4096, "steps": 128, "name": "Qwen3-4B"}),
    "8b": (3, {"num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32,
               "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
               "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
               "tie_word_embeddings": False, "max_position_embeddings": 4096},
           {"batch": 16, "prompt": (64, 2048), "context": 4096, "steps": 256, "name": "Qwen3-8B"}),
    "0.6b": (4, {"num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
                 "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072,
                 "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
                 "tie_word_embeddings": True, "max_position_embeddings": 8192},
             {"batch": 64, "prompt": 7936, "context": 8192, "steps": 64, "name": "Qwen3-0.6B"}),
}
PREFILL_TOKENS = 2048
MIN_TIMED_SECONDS = 1.0
STEP_BUDGET = 900                  # decode steps a timed batch may take in all (keeps its context bucket)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def shape_config(shape: str = "4b"):
    index, preset, _ = SHAPES[shape]
    cfg = dict(preset)
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            text = json.load(f)["configs"][index]
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


def benchmark_config():
    """The default shape (BASELINE.json configs[2])."""
    return shape_config("4b")


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
        time.sleep(0.3)

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


def make_prompts(shape: str, batch: int, vocab: int, seed: int = 0):
    """Uniform random token ids; equal lengths, or seeded uniform lengths for a (low, high) pair."""
    import torch
    _, _, work = SHAPES[shape]
    g = torch.Generator().manual_seed(seed)
    spec = work["prompt"]
    if isinstance(spec, tuple):
        lengths = torch.randint(spec[0], spec[1] + 1, (batch,), generator=g).tolist()
    else:
        lengths = [spec] * batch
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def e2e_new_tokens(steps, context, prompts):
    """New tokens of an end-to-end call, the same for both arms: the timed step count, but no
    fewer than 128 (the longest of the reference's own workloads, bench/bench.py:18-22)."""
    return max(2, min(max(steps, 128), context - max(len(p) for p in prompts)))


def measure_entry(slot, prompt):
    from enginekernel_b200.engine.runner import StepEntry
    return StepEntry(slot, prompt[:PREFILL_TOKENS], [min(len(prompt), PREFILL_TOKENS) - 1])


def timed_generate(engine, prompts, n_new):
    """One whole ``generate`` call on the host's clock: (seconds, seconds to the first token)."""
    import torch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first = None
    for _ in engine.generate(prompts, n_new):
        if first is None:
            first = time.perf_counter()
    torch.cuda.synchronize()
    return time.perf_counter() - t0, first - t0


def end_to_end(engine, prompts, n_new, batch):
    """Whole calls until a second has been timed (three at least); medians."""
    list(engine.generate(prompts, n_new))                              # the shape's graphs exist
    calls, total = [], 0.0
    while len(calls) < 3 or (total < MIN_TIMED_SECONDS and len(calls) < 20):
        whole, ttft = timed_generate(engine, prompts, n_new)
        calls.append((whole, ttft))
        total += whole
    whole = statistics.median(c[0] for c in calls)
    ttft = statistics.median(c[1] for c in calls)
    after_first = statistics.median((c[0] - c[1]) for c in calls)
    return {"value": batch * n_new / whole, "unit": "tok/s", "what": "whole generate() calls: "
            "prompt step and every decode step, host lists in, every step read back",
            "new_tokens": n_new, "calls": len(calls), "call_ms": whole * 1e3, "ttft_ms": ttft * 1e3,
            "after_first_token": batch * (n_new - 1) / after_first if n_new > 1 else None,
            "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4 * batch,
            "prefill_h2d_bytes": 4 * (3 * sum(len(p) for p in prompts) + 2 * batch + 1)}


# --------------------------------------------------------------------------- the reference arm
def run_reference(args) -> int:
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    ref_engine = os.path.join(ROOT, "baseline", "_ref", "engine")
    if not os.path.isfile(os.path.join(ref_engine, "engine.py")):
        return unavailable("baseline/_ref holds no copy of the reference tree (engine/engine.py is missing)")
    if args.gpus != 1:
        return unavailable("the reference runs on one GPU only")
    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device here; the reference arm is timed on a GPU only")
    from enginekernel_b200.config import Qwen3Config
    from enginekernel_b200.weights.random_init import write_random_model

    _, _, work = SHAPES[args.shape]
    raw = shape_config(args.shape)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(raw)
    batch = args.batch or work["batch"]
    steps = args.steps or work["steps"]
    folder = tempfile.mkdtemp(prefix="ek_ref_model_")
    try:
        write_random_model(folder, cfg, seed=0, device="cuda")
        torch.cuda.empty_cache()
        sys.path.insert(0, ref_engine)
        import engine as reference_engine               # the reference's engine/engine.py, unmodified
        eng = reference_engine.Engine(folder)
        prompts = make_prompts(args.shape, batch, cfg.vocab_size)
        n_new = e2e_new_tokens(steps, work["context"], prompts)
        list(eng.generate(prompts, n_new))                # its graphs for this shape are captured here
        for _ in range(max(0, min(args.warmup, 3) - 1)):
            list(eng.generate(prompts, n_new))
        sampler = ClockSampler()
        sampler.start()
        calls, total = [], 0.0
        while len(calls) < 3 or (total < MIN_TIMED_SECONDS and len(calls) < 20):
            whole, ttft = timed_generate(eng, prompts, n_new)
            calls.append((whole, ttft))
            total += whole
        clocks = sampler.stop()
        whole = statistics.median(c[0] for c in calls)
        ttft = statistics.median(c[1] for c in calls)
        after = statistics.median(c[0] - c[1] for c in calls)
        ms_step = after / (n_new - 1) * 1e3
        out = {
            "impl": "reference",
            "metric": f"decode tok/s ({work['name']} shape, batch {batch})",
            "value": batch / (ms_step / 1e3), "unit": "tok/s", "n_gpus": 1, "steps": n_new - 1,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: seeded random weights and uniform random token ids",
            "timing": "host clock between the first token and the end of generate(), device "
                      "synchronised (the reference exposes no device-timed step)",
            "config": {"model": f"{work['name']} shape (Qwen3ForCausalLM)", "shape": args.shape,
                       "num_hidden_layers": full_layers, "layers_run": cfg.num_hidden_layers,
                       "hidden_size": cfg.hidden_size, "vocab_size": cfg.vocab_size,
                       "global_batch": batch, "seq_len": work["context"],
                       "prompt_tokens": sum(len(p) for p in prompts), "parallelism": "none (1 GPU)"},
            "clocks": clocks,
            "e2e": {"value": batch * n_new / whole, "unit": "tok/s", "new_tokens": n_new,
                    "calls": len(calls), "call_ms": whole * 1e3, "ttft_ms": ttft * 1e3,
                    "after_first_token": batch * (n_new - 1) / after},
            "reference": {"tier": getattr(eng, "tier", None),
                          "triton": bool(getattr(eng, "triton", False)) if eng.tier == "fast" else False,
                          "graphs": len(getattr(eng, "graphs", {})) if eng.tier == "fast" else 0,
                          "torch": torch.__version__},
        }
        print(json.dumps(out))
        return 0
    finally:
        shutil.rmtree(folder, ignore_errors=True)


# --------------------------------------------------------------------------- this repository's arm
def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps timed at a stretch (default: the shape's)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="4b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=0, help="sequences in the batch (default: the shape's)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--skip-kernels", action="store_true", help="leave out the per-kernel tables")
    ap.add_argument("--prefill-seqs", type=int, default=1,
                    help="sequences of 2,048 tokens in the prompt step of the per-kernel table")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this library runs on a single B200); --gpus {args.gpus} is not run")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from enginekernel_b200 import Engine, SamplingParams, measure
    from enginekernel_b200.config import Qwen3Config
    from enginekernel_b200.ops.lib import loaded_libraries
    from enginekernel_b200.engine.runner import DEFAULT_MAX_STEP_TOKENS

    _, _, work = SHAPES[args.shape]
    raw = shape_config(args.shape)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(raw)
    pk = peaks()
    batch = args.batch or work["batch"]
    steps = args.steps or work["steps"]
    context = work["context"]
    with_points = args.shape == "4b" and not args.skip_points
    biggest = max(batch, 64 if with_points else 1)
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=biggest * context,
                                max_batch=biggest, max_len=context,
                                max_step_tokens=max(DEFAULT_MAX_STEP_TOKENS, args.prefill_seqs * PREFILL_TOKENS))
    L, H, NH, NKV, D, I, V = (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads,
                              cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size,
                              cfg.vocab_size)
    kv_per_token = 2 * L * NKV * D * 2
    weight_bytes = engine.model.weight_bytes_read_per_step()

    # ---- prefill of 2,048 tokens -------------------------------------------------------
    one = make_prompts("4b", 1, V, seed=1)[0][:PREFILL_TOKENS]
    times = []
    for it in range(4 + 5):                      # 4 warm-ups (clocks, workspace), median of 5
        slot = engine.open_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([(slot, one, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.close_sequence(slot)
        if it >= 4:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)
    per_token_linear = 2 * L * (H * (NH + 2 * NKV) * D + NH * D * H + 3 * H * I)
    attn_flops = L * 4 * NH * D * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2
    prefill_flops = per_token_linear * PREFILL_TOKENS + attn_flops + 2 * H * V
    prefill = {"value": PREFILL_TOKENS / (prefill_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode --------------------------------------------------------------------------
    def decode(b, k, sample_clocks=False, kernels=False):
        """K steps at a stretch, repeated until a second has been timed (or the context is full)."""
        prompts = make_prompts(args.shape, b, V)
        longest = max(len(p) for p in prompts)
        slack = 32                                # steps the per-kernel measurement replays
        room = min(context - longest - warmup - slack, STEP_BUDGET)
        k = max(1, min(k, room))
        run = engine.backend.start(prompts, [warmup + room + slack] * b, SamplingParams(), [],
                                   list(range(b)))
        try:
            st = run.state
            for _ in range(warmup):
                st.step()
            torch.cuda.synchronize()
            sampler = ClockSampler() if sample_clocks else None
            if sampler:
                sampler.start()
            total_ms, repeats, done = 0.0, 0, warmup
            while repeats == 0 or (total_ms < MIN_TIMED_SECONDS * 1e3 and done + k <= room + warmup):
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(k):
                    st.step()
                e.record()
                torch.cuda.synchronize()
                total_ms += a.elapsed_time(e)
                repeats += 1
                done += k
            clocks = sampler.stop() if sampler else None
            ms = total_ms / (repeats * k)
            mean_context = sum(len(p) for p in prompts) / b + warmup + (done - warmup) / 2
            table = None
            if kernels:
                table = measure.decode_step_table(st, pk)
                table["batch"], table["context"] = b, int(mean_context + (done - warmup) / 2)
            return {"ms": ms, "clocks": clocks, "launches": st.launches_per_step, "repeats": repeats,
                    "steps": k, "mean_context": mean_context, "kernels": table}
        finally:
            run.close()

    main_run = decode(batch, steps, sample_clocks=True, kernels=not args.skip_kernels)
    ms_step = main_run["ms"]
    value = batch / (ms_step / 1e3)
    step_bytes = weight_bytes + batch * main_run["mean_context"] * kv_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}

    points, point_fracs = {}, {}
    if with_points:
        for b in (1, 64):
            r = decode(b, max(16, steps // 2))
            points[f"decode_b{b}"] = b / (r["ms"] / 1e3)
            bytes_b = weight_bytes + b * r["mean_context"] * kv_per_token
            point_fracs[f"decode_b{b}"] = bytes_b / (r["ms"] / 1e3) / 1e9 / pk["hbm_gbs"]

    kernels = {}
    if main_run["kernels"] is not None:
        kernels["decode"] = main_run["kernels"]
        n_pre = max(1, min(args.prefill_seqs, biggest))
        many = make_prompts("4b", n_pre, V, seed=1)
        slots = [engine.open_sequence() for _ in many]
        try:
            kernels["prefill"] = measure.prefill_step_table(
                lambda: engine.runner.step([measure_entry(s, p) for s, p in zip(slots, many)]), pk)
            kernels["prefill"]["tokens"] = n_pre * PREFILL_TOKENS
        finally:
            for s in slots:
                engine.close_sequence(s)

    # ---- end to end through Engine.generate --------------------------------------------
    host_prompts = make_prompts(args.shape, batch, V)
    n_new = e2e_new_tokens(steps, context, host_prompts)
    e2e = end_to_end(engine, host_prompts, n_new, batch)

    prompt_desc = work["prompt"]
    out = {
        "metric": f"decode tok/s ({work['name']} shape, batch {batch}, "
                  + (f"{prompt_desc[0]}-{prompt_desc[1]}-token prompts)" if isinstance(prompt_desc, tuple)
                     else f"{prompt_desc:,}-token prompts)"),
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": main_run["steps"], "warmup": warmup,
        "repeats": main_run["repeats"], "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {
            "model": f"{work['name']} shape (Qwen3ForCausalLM)", "shape": args.shape,
            "num_hidden_layers": full_layers, "layers_run": cfg.num_hidden_layers, "hidden_size": H,
            "num_attention_heads": NH, "num_key_value_heads": NKV, "head_dim": D,
            "intermediate_size": I, "vocab_size": V, "tie_word_embeddings": cfg.tie_word_embeddings,
            "rope_theta": cfg.rope_theta, "global_batch": batch, "seq_len": context,
            "prompt_len": prompt_desc if not isinstance(prompt_desc, tuple) else
            int(sum(len(p) for p in host_prompts) / batch),
            "parallelism": "none (1 GPU)",
            "l2": "step inputs (gigabytes of weights and cache) exceed the 126 MB L2",
            "peaks": pk["source"]},
        "clocks": main_run["clocks"], "e2e": e2e,
        "gpu_launches": main_run["launches"] * main_run["steps"] * main_run["repeats"],
        "prefill": prefill, "roofline": roofline, "points": points, "point_fracs": point_fracs,
        "kernels": kernels,
        "kernel_libraries": sorted(os.path.basename(p) for p in loaded_libraries().values()),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
