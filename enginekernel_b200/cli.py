"""Command line: token ids in, token ids out.

    python -m enginekernel_b200 generate --model DIR --batch 4 --in-len 512 --out-len 32
    python -m enginekernel_b200 generate --model DIR --prompt-ids "5,17,3;9,9" --out-len 8 --temperature 0.8
    python -m enginekernel_b200 random-model --config config.json --seed 0 --out DIR
    python -m enginekernel_b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl

Option names follow the reference's scripts where it has them: ``--model``, ``--batch``,
``--in-len``, ``--out-len``, ``--mode`` (bench/check_exact.py:73-79), ``--samples``
(bench/bench.py:42-47).  ``--mode random`` draws uniform token ids with seed 0 as the reference
does (bench/bench.py:25-27); its ``text`` mode needs a tokenizer and a corpus and is not offered.
Like the reference, nothing here tokenises.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
import time


def _parse_prompts(args, vocab):
    if args.prompt_ids:
        return [[int(t) for t in row.split(",") if t.strip()] for row in args.prompt_ids.split(";")]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            data = json.load(f)
        return [[int(t) for t in row] for row in data]
    import torch
    g = torch.Generator().manual_seed(args.prompt_seed)
    return torch.randint(0, vocab, (args.batch, args.in_len), generator=g).tolist()


def cmd_generate(args) -> int:
    from .engine.engine import Engine
    from .registry import config_from_folder, model_spec_for
    t0 = time.perf_counter()
    prompts = _parse_prompts(args, model_spec_for(config_from_folder(args.model)).vocab_size)
    # the cache holds every prompt with its output, each counted in whole pages of 64 tokens
    need = sum(64 * ((len(p) + args.out_len) // 64 + 1) for p in prompts)
    engine = Engine(args.model, args.dtype, max_tokens=max(args.max_tokens or 0, need),
                    max_batch=args.max_batch or max(len(prompts), 1))
    print(f"engine load: {time.perf_counter() - t0:.1f}s", file=sys.stderr)
    kw = dict(temperature=args.temperature, top_k=args.top_k, seed=args.seed,
              stop_token_ids=[int(s) for s in args.stop_ids.split(",") if s.strip()])
    times, ttfts, out = [], [], None
    for sample in range(max(1, args.samples)):
        t0 = time.perf_counter()
        ttft = None
        out = [[] for _ in prompts]
        if len(prompts) <= engine.backend.max_batch:
            for step in engine.generate(prompts, args.out_len, **kw):
                if ttft is None:
                    ttft = time.perf_counter() - t0
                for row, tok in zip(out, step):
                    if tok >= 0:
                        row.append(tok)
        else:
            out = engine.generate_all(prompts, args.out_len, **kw)
        times.append(time.perf_counter() - t0)
        ttfts.append(ttft or times[-1])
    for i, row in enumerate(out):
        print(json.dumps({"request": i, "tokens": row}))
    med = statistics.median(times)
    n = sum(len(r) for r in out)
    print(f"{n / med:8.1f} tok/s  median {med * 1000:7.1f}ms  ttft {statistics.median(ttfts) * 1000:6.1f}ms  "
          f"spread {(max(times) - min(times)) / med * 100:4.1f}%", file=sys.stderr)
    return 0


def cmd_random_model(args) -> int:
    import torch
    from .registry import architecture_of, lookup_architecture
    from .weights.random_init import write_random_model
    with open(args.config) as f:
        raw = json.load(f)
    config_cls, _ = lookup_architecture(architecture_of(raw))
    cfg = config_cls.from_dict(raw)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    print(write_random_model(args.out, cfg, args.seed, dtype))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="enginekernel_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids from prompts of token ids")
    g.add_argument("--model", required=True, help="folder with config.json and safetensors")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--batch", type=int, default=1, help="number of random prompts (--mode random)")
    g.add_argument("--in-len", type=int, default=512, help="length of the random prompts")
    g.add_argument("--out-len", type=int, default=32, help="tokens to generate per request")
    g.add_argument("--mode", default="random", choices=["random"],
                   help="where prompts come from when no ids are given")
    g.add_argument("--prompt-ids", default="", help='explicit prompts: "1,2,3;4,5"')
    g.add_argument("--prompt-file", default="", help="JSON file: list of lists of token ids")
    g.add_argument("--prompt-seed", type=int, default=0)
    g.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    g.add_argument("--top-k", type=int, default=0, help="0: no restriction")
    g.add_argument("--seed", type=int, default=0, help="sampling seed")
    g.add_argument("--stop-ids", default="", help="comma-separated token ids that end a sequence")
    g.add_argument("--samples", type=int, default=1, help="timed repetitions")
    g.add_argument("--max-tokens", type=int, default=0, help="cache size in tokens")
    g.add_argument("--max-batch", type=int, default=0, help="most sequences per batch")
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_random_model)

    p = sub.add_parser("replay", help="trace replay (same options as bin/trace_run)", add_help=False)
    p.set_defaults(fn=None)

    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .replay import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
