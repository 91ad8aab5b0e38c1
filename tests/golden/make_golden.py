"""Make the golden outputs that anchor the plain implementation on the reference.

Runs the reference's own model code (engine/ek_model.py of the reference project)
on the CPU in float32 for the tiny configurations A and B with seeded random
weights, and stores logits at every position of a few prompts.  The reference is
imported with its Triton path disabled (environment variable ENGINE_NO_TRITON=1 set
before the import), so only its torch formulas run.  Logits at position n-1 come
from ``prefill`` of the first n tokens; the last rows also from ``prefill`` of one
token followed by ``decode`` steps, which exercises its cache path.

    python tests/golden/make_golden.py /path/to/reference

Outputs: tests/golden/tiny_a.pt, tests/golden/tiny_b.pt (a few hundred KB each).
"""

from __future__ import annotations

import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.plain import tiny_models  # noqa: E402


def reference_logits(ref_model, ids):
    c = ref_model.cfg
    rows = []
    for n in range(1, len(ids) + 1):
        k = [torch.zeros(1, c.num_kv_heads, n, c.head_dim) for _ in range(c.num_layers)]
        v = [torch.zeros(1, c.num_kv_heads, n, c.head_dim) for _ in range(c.num_layers)]
        t = torch.tensor([ids[:n]])
        pos = torch.arange(n)[None]
        hidden = ref_model.prefill(t, pos, k, v)
        rows.append(hidden @ ref_model.lm_head_t)
    return torch.cat(rows, 0)


def reference_decode_logits(ref_model, ids):
    """One-token prefill, then the reference's decode() for every further token."""
    c = ref_model.cfg
    n = len(ids)
    k = [torch.zeros(1, c.num_kv_heads, n, c.head_dim) for _ in range(c.num_layers)]
    v = [torch.zeros(1, c.num_kv_heads, n, c.head_dim) for _ in range(c.num_layers)]
    hidden = ref_model.prefill(torch.tensor([ids[:1]]), torch.zeros(1, 1, dtype=torch.long), k, v)
    rows = [hidden @ ref_model.lm_head_t]
    slot_t = torch.zeros(1, dtype=torch.int64)
    len_t = torch.full((1,), 1, dtype=torch.int64)
    start_t = torch.zeros(1, dtype=torch.int32)
    for j in range(1, n):
        hidden = ref_model.decode(torch.tensor([ids[j]]), torch.tensor([j]), k, v,
                                  slot_t, len_t, start_t, None)
        rows.append(hidden @ ref_model.lm_head_t)
    return torch.cat(rows, 0)


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of jeojdi1/EngineKernel>")
    ref_root = sys.argv[1]
    os.environ["ENGINE_NO_TRITON"] = "1"
    sys.path.insert(0, os.path.join(ref_root, "engine"))
    import ek_model  # the reference's module

    for tag, cfg, seed, lengths in (("tiny_a", tiny_models.TINY_A, 0, (5, 9, 13)),
                                    ("tiny_b", tiny_models.TINY_B, 1, (1, 7, 16, 31))):
        with tempfile.TemporaryDirectory() as tmp:
            tiny_models.write_tiny(tmp, cfg, seed, dtype=torch.float32)
            ref = ek_model.Qwen3(tmp, torch.device("cpu"), dtype=torch.float32)
            prompts = tiny_models.random_prompts(cfg, lengths, seed=100 + seed)
            with torch.inference_mode():
                out = {"config": cfg, "weight_seed": seed, "prompts": prompts,
                       "prefill_logits": [reference_logits(ref, p).clone() for p in prompts],
                       "decode_logits": [reference_decode_logits(ref, p).clone() for p in prompts]}
        torch.save(out, os.path.join(HERE, tag + ".pt"))
        print(tag, [tuple(t.shape) for t in out["prefill_logits"]])


if __name__ == "__main__":
    main()
