"""y = x . W^T for the engine's two precisions.

* float32: the hand-written FFMA kernel (no tensor-core mode of reduced precision).
* bfloat16, at most 64 rows (decode): the tcgen05 kernel in its swapped form - weights on the
  128-row side of the MMA, TMA-streamed, K split over blocks.
* bfloat16, more rows (prefill): the tcgen05 kernel on pairs of SMs (256 x 256 tiles, a
  persistent launch) where its tiles fill the GPU's pairs evenly, with the residual add or
  SwiGLU in its epilogue; else the library product, where the reference also calls a
  library (``torch.matmul`` on cuBLAS, engine/ek_model.py:298,311,203-209).
"""

from __future__ import annotations

import torch

from . import kernels, lib

SMALL_ROWS = kernels.TC_SWAP_MAX_ROWS


def tc_takes(x, w) -> bool:
    """Whether the tcgen05 kernel can read these operands (16-byte aligned rows)."""
    return (w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


DEFER_NORM_ROWS = 16      # measured on the Qwen3-4B shape: +2.3 % at 1 row, even at 8, -3.6 % at 64


def can_defer_norm(ctx, w, n_rows) -> bool:
    """Whether products of this step carry a deferred norm: the bfloat16 path with few rows (the
    swapped tcgen05 form at its narrowest tile, where a norm kernel of its own is all latency),
    weights TMA can address."""
    return (w.dtype == torch.bfloat16 and n_rows <= DEFER_NORM_ROWS and w.shape[1] % 8 == 0
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)


def row_scale_of(deferred):
    return deferred.ss, deferred.size, deferred.eps


PAIR_MIN_FILL = 0.8       # of the last wave of tiles; below it the library's smaller tiles win
PAIR_ADDS_TO_STREAM = False


def pair_fill(m, n_tiles_n, device) -> float:
    """How evenly the pair product's tiles fill the GPU: tiles / (waves * pairs of SMs)."""
    tiles = -(-m // 256) * n_tiles_n
    pairs = max(1, kernels.sm_count(device) // 2)
    return tiles / (-(-tiles // pairs) * pairs)


def pair_product_wins(out, x, w, m, epilogue) -> bool:
    """Whether a product of ``m`` rows goes to the kernel on pairs of SMs.  Its plain and its adding
    form run at the library's speed launch by launch (0.96-1.02 of it), and a long prompt step is
    bound by the power cap, where the library's adding product came out ahead (8 x 2,048 tokens of
    the Qwen3-4B shape: 111.3 ms a step with the library adding, 113.2 ms with this kernel, 117.5 ms
    with the library for every product); so the kernel takes the products whose epilogue saves a
    kernel and a round trip through memory - SwiGLU, and q/k/v with norm, rotation and cache write -
    and the library the ones that add to the stream."""
    if epilogue == kernels.PAIR_EPI_ADD_F32 and not PAIR_ADDS_TO_STREAM:
        return False
    if m <= SMALL_ROWS or not kernels.gemm_pair_takes(out, x, w, epilogue):
        return False
    n = w.shape[0]
    n_tiles = -(-(n // 2) // 128) if epilogue == kernels.PAIR_EPI_SWIGLU else -(-n // 256)
    return pair_fill(m, n_tiles, x.device) >= PAIR_MIN_FILL


def linear(x, w, ctx, name: str, n_rows=None, out_dtype=None, defer=None):
    """``x`` [M, K] (dense rows), ``w`` [N, K] -> [M, N] from the step's workspace.

    ``x`` may be a :class:`~enginekernel_b200.parts.base.DeferredNorm` (the product scales its
    rows).  ``defer=(stream, norm)``: the caller will add the result to ``stream`` and apply
    ``norm`` next, and this product may do part of that: with few rows the result is added to
    ``stream`` here and a DeferredNorm for ``norm`` is returned; with many rows (bfloat16) the
    product adds its 32-bit result to ``stream`` and None is returned (nothing left to add: the
    norm is called without ``add``).  Otherwise the plain result comes back."""
    from ..parts.base import DeferredNorm
    row_scale = None
    if isinstance(x, DeferredNorm):
        row_scale, x = row_scale_of(x), x.scaled
    m = n_rows if n_rows is not None else x.shape[0]
    n = w.shape[0]
    if defer is not None:
        stream, norm = defer
        spec = norm.deferrable()
        if (spec is not None and out_dtype is None and can_defer_norm(ctx, w, m) and tc_takes(x, w)
                and n % 8 == 0 and spec[0].numel() == n and stream.shape[-1] == n):
            gain, eps = spec
            tiles = -(-n // 128)
            scaled = ctx.workspace.get("deferred_" + name, (m, n), torch.bfloat16)
            ss = ctx.workspace.get("deferred_ss_" + name, (m, tiles), torch.float32)
            kernels.gemm_tc_bf16(scaled, x, w, kernels.EPI_BF16, n_rows=m, swap=True,
                                 row_scale=row_scale, residual=(stream, gain, ss))
            return DeferredNorm(scaled, ss, tiles, n, float(eps))
    if (defer is not None and row_scale is None and out_dtype is None and w.dtype == torch.bfloat16
            and m > SMALL_ROWS):
        # many rows (a prompt): the product adds its 32-bit result to the stream itself
        # (bfloat16 operands, 32-bit C and D), so the norm that follows only reads the stream
        stream = defer[0]
        if stream.dtype == torch.float32 and stream.shape[-1] == n and stream.is_contiguous() \
                and stream.shape[0] >= m:
            if pair_product_wins(stream, x, w, m, kernels.PAIR_EPI_ADD_F32):
                kernels.gemm_pair_bf16(stream, x, w, kernels.PAIR_EPI_ADD_F32, n_rows=m)
            else:
                _library_product_add(stream[:m], x[:m], w)
            return None
    if row_scale is not None and not (w.dtype == torch.bfloat16 and m <= SMALL_ROWS and tc_takes(x, w)):
        raise kernels.KernelError("a deferred norm reached a product that cannot scale its rows")
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
            _library_product(x[:m].float(), w.float(), out)
        else:
            _library_product(x[:m], w, out)
        return out
    if m <= SMALL_ROWS:
        kernels.gemm_tc_bf16(out, x, w, epi, n_rows=m, swap=True, row_scale=row_scale)
    elif want_f32:
        # 32-bit logits for many rows: 128 x 128 tiles with the accumulator stored as it is
        kernels.gemm_tc_bf16(out, x, w, epi, n_rows=m, swap=False)
    elif pair_product_wins(out, x, w, m, kernels.PAIR_EPI_BF16):
        kernels.gemm_pair_bf16(out, x, w, kernels.PAIR_EPI_BF16, n_rows=m)
    else:
        _library_product(x[:m], w, out)
    return out


def _library_product_add(stream, x, w):
    """stream += x . w^T by the library, accumulated and added in 32-bit (no rounding of the
    product to 16 bits on its way into the residual stream)."""
    torch.addmm(stream, x, w.t(), out_dtype=torch.float32, out=stream)
    if lib.recording():
        m, k = x.shape
        n = w.shape[0]
        lib.record_library_call(f"library_addmm[{n}x{k}]",
                                lambda: torch.addmm(stream, x, w.t(), out_dtype=torch.float32, out=stream),
                                bytes=x.element_size() * (m * k + n * k) + 8 * m * n, flops=2 * m * n * k)


def _library_product(x, w, out):
    """out = x . w^T by the library (cuBLAS through torch), as the reference does for prompts
    (engine/ek_model.py:298, 311, 203-209)."""
    torch.matmul(x, w.t(), out=out)
    if lib.recording():
        m, k = x.shape
        n = w.shape[0]
        lib.record_library_call(f"library_matmul[{n}x{k}]", lambda: torch.matmul(x, w.t(), out=out),
                                bytes=x.element_size() * (m * k + n * k) + out.element_size() * m * n,
                                flops=2 * m * n * k)
