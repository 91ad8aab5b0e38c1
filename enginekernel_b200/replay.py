"""Trace replay: feed given token ids through the model step by step and write logits.

Reads one JSON object per line from standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Each entry gives a request's next tokens and the places among them whose logits are
wanted; ``end`` lists requests that are finished after the step (what they hold is given
back).  For a step that wants something, ``<out>/<step>.f32`` receives the logits as
little-endian 32-bit floats [wanted, vocab], in the order of the entries and of ``want``.
After every step ``done <step>`` is printed and flushed.  Nothing is sampled.  The tool
drives the same model, step function, cache and kernels as generation; it has none of its
own.  (The reference's nearest tool teacher-forces tokens through another library and
compares arg-max margins, bench/check_exact.py:45-69.)
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at once, each rounded up to 64")
    args = ap.parse_args(argv)

    from .cache.pages import PAGE
    from .engine.engine import Engine
    from .engine.runner import StepEntry

    os.makedirs(args.out, exist_ok=True)
    max_tokens = max(PAGE, -(-args.max_tokens // PAGE) * PAGE)
    engine = Engine(args.model, args.dtype, max_tokens=max_tokens,
                    max_batch=max(1, max_tokens // PAGE))
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for e in step.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.open_sequence()
            entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        logits = engine.runner.step(entries)          # a view, written to the file before the next step
        if logits.shape[0] > 0:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            path = os.path.join(args.out, f"{step['step']}.f32")
            with open(path + ".tmp", "wb") as f:
                f.write(arr.tobytes())
            os.replace(path + ".tmp", path)
        engine.runner.check_kernels()
        for rid in step.get("end", []):
            if rid in slots:
                engine.close_sequence(slots.pop(rid))
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
