"""y = x . W^T for the engine's two precisions.

* float32: the hand-written FFMA kernel (no tensor-core mode of reduced precision).
* bfloat16, at most 64 rows (decode): the tcgen05 kernel in its swapped form - weights on the
  128-row side of the MMA, TMA-streamed, K split over blocks.
* bfloat16, more rows (prefill): the library product, where the reference also calls a
  library (``torch.matmul`` on cuBLAS, engine/ek_model.py:298,311,203-209).
"""

from __future__ import annotations

import torch

from . import kernels

SMALL_ROWS = kernels.TC_SWAP_MAX_ROWS


def tc_takes(x, w) -> bool:
    """Whether the tcgen05 kernel can read these operands (16-byte aligned rows)."""
    return (w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear(x, w, ctx, name: str, n_rows=None, out_dtype=None):
    """``x`` [M, K] (dense rows), ``w`` [N, K] -> [M, N] from the step's workspace."""
    m = n_rows if n_rows is not None else x.shape[0]
    n = w.shape[0]
    if w.dtype == torch.float32:
        out = ctx.workspace.get(name, (m, n), torch.float32)
        kernels.gemm_f32(out, x, w, n_rows=m)
        return out
    want_f32 = out_dtype == torch.float32
    epi = kernels.EPI_F32 if want_f32 else kernels.EPI_BF16
    out = ctx.workspace.get(name, (m, n), torch.float32 if want_f32 else torch.bfloat16)
    if not tc_takes(x, w):
        # rows that TMA cannot address (inner size or stride not a multiple of 8 values): the
        # library product, rounded once from its 32-bit accumulator
        if want_f32:
            torch.matmul(x[:m].float(), w.float().t(), out=out)
        else:
            torch.matmul(x[:m], w.t(), out=out)
        return out
    if m <= SMALL_ROWS:
        kernels.gemm_tc_bf16(out, x, w, epi, n_rows=m, swap=True)
    elif want_f32:
        # 32-bit logits for many rows: 128 x 128 tiles with the accumulator stored as it is
        kernels.gemm_tc_bf16(out, x, w, epi, n_rows=m, swap=False)
    else:
        torch.matmul(x[:m], w.t(), out=out)
    return out
