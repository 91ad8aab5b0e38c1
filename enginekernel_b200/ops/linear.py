"""y = x . W^T for the engine's two precisions.

* float32: the hand-written FFMA kernel (no tensor-core mode of reduced precision).
* bfloat16, at most 64 rows (decode): the weight-streaming tensor-core kernel.
* bfloat16, more rows (prefill): the library product, where the reference also calls a
  library (``torch.matmul`` on cuBLAS, engine/ek_model.py:298,311,203-209).
"""

from __future__ import annotations

import torch

from . import kernels


def linear(x, w, ctx, name: str, n_rows=None, out_dtype=None):
    """``x`` [M, K] (dense rows), ``w`` [N, K] -> [M, N] from the step's workspace."""
    m = n_rows if n_rows is not None else x.shape[0]
    n = w.shape[0]
    if w.dtype == torch.float32:
        out = ctx.workspace.get(name, (m, n), torch.float32)
        kernels.gemm_f32(out, x, w, n_rows=m)
        return out
    want_f32 = out_dtype == torch.float32
    if m <= kernels.GEMV_MAX_ROWS:
        out = ctx.workspace.get(name, (m, n), torch.float32 if want_f32 else torch.bfloat16)
        kernels.gemv_bf16(out, x, w, kernels.EPI_F32 if want_f32 else kernels.EPI_BF16, n_rows=m)
        return out
    if want_f32:
        out = ctx.workspace.get(name, (m, n), torch.float32)
        for r0 in range(0, m, kernels.GEMV_MAX_ROWS):
            r1 = min(m, r0 + kernels.GEMV_MAX_ROWS)
            kernels.gemv_bf16(out[r0:r1], x[r0:r1], w, kernels.EPI_F32, n_rows=r1 - r0)
        return out
    out = ctx.workspace.get(name, (m, n), torch.bfloat16)
    torch.matmul(x[:m], w.t(), out=out)
    return out
