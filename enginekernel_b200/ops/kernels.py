"""Python faces of the CUDA kernels: argument checks, then one launch each.

Every function takes CUDA tensors and launches on torch's current stream.  There is
no CPU or torch fallback: a tensor that is not on a CUDA device, or a kernel library
that cannot be built or loaded, raises.  The reference pairs every Triton kernel with
a torch fallback chosen at call time (engine/ek_kernels.py:1025-1559); here the plain
counterparts live only in the tests.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import lib
from .lib import Function, KernelError, count_extra_launches

PAGE = 64                 # tokens per cache page; must equal EK_PAGE in csrc/common.cuh
MAX_HEAD_DIM = 256

_SUFFIX = {torch.float32: "f32", torch.bfloat16: "bf16"}
_P = c_void_p


def _suffix(dtype) -> str:
    try:
        return _SUFFIX[dtype]
    except KeyError:
        raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}") from None


def _ptr(t):
    return None if t is None else t.data_ptr()


def _slow_stream():
    return torch.cuda.current_stream().cuda_stream


# The handle of torch's current stream on the current device.  The public way costs the host 3 us
# a launch (a Stream object is built each time); torch's own raw accessors, where this build of
# torch has them, a tenth of that.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is None or _raw_device is None:
        return _slow_stream()
    return _raw_stream(_raw_device())


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("enginekernel_b200 kernels run on CUDA tensors only; got a tensor on "
                              f"{t.device} (there is no CPU path)")


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _attention_cost(q, n_tokens, positions, n_q_heads, n_kv_heads, head_dim, window, new_keys_only):
    """While a launch record is active: what an attention launch has to read and compute.  Reads
    the positions back (a synchronisation, which is why it is done only then).  Keys and values:
    for single tokens every visible key of every token; for prompts (``new_keys_only``) each
    token's own key and value once, as the work is bound by its flops anyway."""
    if not lib.recording():
        return
    pos = positions[:n_tokens].to(torch.int64)
    visible = torch.clamp(pos + 1, min=0)
    if window:
        visible = torch.clamp(visible, max=int(window))
    keys = int(visible.sum().item())
    live = int((pos >= 0).sum().item())
    size = q.element_size()
    kv_tokens = live if new_keys_only else keys
    lib.annotate(bytes=size * (2 * kv_tokens * n_kv_heads * head_dim + 2 * live * n_q_heads * head_dim),
                 flops=4 * keys * n_q_heads * head_dim)


def _per_dtype(module, name, argtypes):
    return {dt: Function(module, f"{name}_{sfx}", argtypes) for dt, sfx in _SUFFIX.items()}


# ------------------------------------------------------------------ elementwise
_embed = _per_dtype("elementwise", "ek_embed", [_P, _P, _P, c_int, c_int, c_int, c_float, _P, _P, c_int, _P])
_scale_f32 = Function("elementwise", "ek_scale_f32", [_P, c_longlong, c_float, _P])
_rmsnorm = _per_dtype("elementwise", "ek_rmsnorm",
                      [_P, _P, _P, _P, _P, c_float, c_int, c_int, c_int, _P])
_add_residual = _per_dtype("elementwise", "ek_add_residual", [_P, _P, c_longlong, _P])
_silu_mul = _per_dtype("elementwise", "ek_silu_mul", [_P, _P, c_int, c_int, _P])


def embed(resid, table, ids, n_tokens, scale=1.0, pos_table=None, positions=None):
    """resid[t, :] = table[ids[t], :] * scale as 32-bit, for the first ``n_tokens`` ids; with
    ``pos_table`` [positions, hidden] also + pos_table[positions[t], :] (rows whose position is
    negative get none).  A plain launch: the first kernel of a step."""
    _need_cuda(resid, table, ids, pos_table, positions)
    _need(resid.dtype == torch.float32 and ids.dtype == torch.int32, "embed: resid f32, ids int32")
    _need(table.is_contiguous() and resid.is_contiguous(), "embed: contiguous tensors")
    vocab, hidden = table.shape
    _need(resid.shape[-1] == hidden and resid.shape[0] >= n_tokens, "embed: resid shape")
    max_positions = 0
    if pos_table is not None:
        _need(pos_table.dtype == table.dtype and pos_table.is_contiguous() and pos_table.shape[-1] == hidden
              and positions is not None and positions.dtype == torch.int32,
              "embed: position table [positions, hidden] in the embedding's dtype, int32 positions")
        max_positions = pos_table.shape[0]
    if lib.recording():
        lib.annotate(bytes=n_tokens * hidden * (table.element_size() * (2 if pos_table is not None else 1) + 4))
    _embed[table.dtype](_ptr(resid), _ptr(table), _ptr(ids), n_tokens, hidden, vocab, float(scale),
                        _ptr(pos_table), _ptr(positions), max_positions, _stream())


def scale_(x, scale, n=None):
    """x *= scale in place (32-bit values; the first ``n`` of them)."""
    _need_cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "scale_: contiguous 32-bit values")
    count = x.numel() if n is None else n
    if lib.recording():
        lib.annotate(bytes=8 * count)
    _scale_f32(_ptr(x), count, float(scale), _stream())


def rmsnorm(y, resid, gain, eps, add=None, rows=None, n_rows=None, write_back=True):
    """y = gain * n(resid [+ add]); with ``add`` the stream is updated in place when
    ``write_back``.  ``rows`` (int32) picks stream rows; y then has one row per entry."""
    _need_cuda(y, resid, gain, add, rows)
    hidden = resid.shape[-1]
    _need(resid.dtype == torch.float32 and gain.dtype == torch.float32, "rmsnorm: 32-bit stream and gain")
    _need(gain.numel() == hidden and y.shape[-1] == hidden, "rmsnorm: sizes disagree")
    _need(add is None or (add.dtype == y.dtype and add.shape[-1] == hidden and add.is_contiguous()),
          "rmsnorm: add must have y's dtype and the stream's width")
    _need(y.is_contiguous() and resid.is_contiguous(), "rmsnorm: contiguous tensors")
    if n_rows is None:
        n_rows = rows.numel() if rows is not None else resid.shape[0]
    _need(y.shape[0] >= n_rows, "rmsnorm: y has too few rows")
    if lib.recording():
        per_value = 4 + y.element_size() + ((y.element_size() + (4 if write_back else 0)) if add is not None else 0)
        lib.annotate(bytes=n_rows * hidden * per_value)
    _rmsnorm[y.dtype](_ptr(y), _ptr(resid), _ptr(add), _ptr(gain), _ptr(rows), float(eps),
                      n_rows, hidden, 1 if write_back else 0, _stream())


def add_residual(resid, x, n_rows=None):
    _need_cuda(resid, x)
    n = (n_rows if n_rows is not None else resid.shape[0]) * resid.shape[-1]
    _need(resid.dtype == torch.float32 and x.shape[-1] == resid.shape[-1], "add_residual: shapes")
    _add_residual[x.dtype](_ptr(resid), _ptr(x), n, _stream())


def silu_mul(out, gu, n_rows=None):
    """out[r, i] = silu(gu[r, i]) * gu[r, I + i] for gu of width 2I."""
    _need_cuda(out, gu)
    inter = gu.shape[-1] // 2
    _need(gu.shape[-1] == 2 * inter and out.shape[-1] == inter and out.dtype == gu.dtype,
          "silu_mul: out must be [rows, I] for gu [rows, 2I]")
    _need(out.is_contiguous() and gu.is_contiguous(), "silu_mul: contiguous tensors")
    rows = n_rows if n_rows is not None else gu.shape[0]
    if lib.recording():
        lib.annotate(bytes=3 * rows * inter * gu.element_size())
    for r0 in range(0, rows, 65535):
        r1 = min(rows, r0 + 65535)
        _silu_mul[gu.dtype](_ptr(out[r0:]), _ptr(gu[r0:]), r1 - r0, inter, _stream())


# ------------------------------------------------------------------ rope + cache write
_rope_kv = _per_dtype("rope_kv", "ek_qk_norm_rope_kv",
                      [_P, c_int, _P, _P, _P, _P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int,
                       c_int, c_int, c_float, c_int, _P])


def check_head_dim(head_dim):
    if head_dim % 16 or not 16 <= head_dim <= MAX_HEAD_DIM:
        raise KernelError(f"head size {head_dim} is not supported: the attention kernels take "
                          f"multiples of 16 from 16 to {MAX_HEAD_DIM}")


def qk_norm_rope_kv(qkv, n_tokens, q_gain, k_gain, cos, sin, rot_dim, positions, token_slot,
                    k_pages, v_pages, block_table, n_q_heads, n_kv_heads, head_dim, eps,
                    write_kv=True):
    """In place on the q part of ``qkv`` [T, (NQ + 2 NKV) D]; keys and values go to the pages."""
    _need_cuda(qkv, cos, sin, positions, token_slot, k_pages, v_pages, block_table)
    check_head_dim(head_dim)
    _need(qkv.stride(-1) == 1 and qkv.shape[-1] == (n_q_heads + 2 * n_kv_heads) * head_dim,
          "qk_norm_rope_kv: qkv width")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
          and cos.shape[-1] * 2 == rot_dim, "qk_norm_rope_kv: 32-bit tables of rot_dim/2 columns")
    _need(k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype, "qk_norm_rope_kv: cache dtype")
    _need(block_table.dtype == torch.int32 and positions.dtype == torch.int32
          and token_slot.dtype == torch.int32, "qk_norm_rope_kv: int32 indices")
    for g in (q_gain, k_gain):
        _need(g is None or (g.dtype == torch.float32 and g.numel() == head_dim), "qk gains: 32-bit [D]")
    if lib.recording():
        lib.annotate(bytes=n_tokens * head_dim * qkv.element_size() * (2 * n_q_heads + 3 * n_kv_heads))
    _rope_kv[qkv.dtype](_ptr(qkv), qkv.stride(0), _ptr(q_gain), _ptr(k_gain), _ptr(cos), _ptr(sin),
                        rot_dim, _ptr(positions), _ptr(token_slot), _ptr(k_pages), _ptr(v_pages),
                        _ptr(block_table), block_table.stride(0), n_tokens, n_q_heads, n_kv_heads,
                        head_dim, float(eps), 1 if write_kv else 0, _stream())


# ------------------------------------------------------------------ attention
_attn_generic = _per_dtype("attention_generic", "ek_attention_generic",
                           [_P, _P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                            c_float, c_int, c_int, c_int, _P, _P, _P])


def attention_generic(out, q, n_tokens, positions, token_slot, k_pages, v_pages, block_table,
                      n_q_heads, n_kv_heads, head_dim, scale, window=None, n_splits=1,
                      keys_per_split=0, part_acc=None, part_ml=None):
    """out[t, h*D:(h+1)*D] = softmax(scale q.K^T) V over the keys token t may see.

    ``q`` is any tensor whose row t starts with the NQ*D query values (the fused q/k/v
    rows qualify).  With ``n_splits`` > 1 the keys are cut every ``keys_per_split`` and
    merged from ``part_acc`` [T, NQ, splits, D] / ``part_ml`` [T, NQ, splits, 2] (32-bit).
    """
    _need_cuda(out, q, positions, token_slot, k_pages, v_pages, block_table, part_acc, part_ml)
    check_head_dim(head_dim)
    _need(out.dtype == q.dtype == k_pages.dtype, "attention: one dtype for q, cache and out")
    _need(out.is_contiguous() and out.shape[-1] == n_q_heads * head_dim, "attention: out [T, NQ*D]")
    _need(q.stride(-1) == 1, "attention: q rows must be dense")
    if n_splits > 1:
        _need(part_acc is not None and part_ml is not None
              and part_acc.numel() >= n_tokens * n_q_heads * n_splits * head_dim
              and part_ml.numel() >= n_tokens * n_q_heads * n_splits * 2, "attention: split buffers")
    _attention_cost(q, n_tokens, positions, n_q_heads, n_kv_heads, head_dim, window, False)
    _attn_generic[q.dtype](_ptr(out), _ptr(q), q.stride(0), _ptr(positions), _ptr(token_slot),
                           _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.stride(0),
                           n_tokens, n_q_heads, n_kv_heads, head_dim, float(scale),
                           int(window or 0), n_splits, keys_per_split, _ptr(part_acc),
                           _ptr(part_ml), _stream())
    if n_splits > 1:
        count_extra_launches()               # the merge kernel


_attn_decode_bf16 = Function("attention_decode_bf16", "ek_attention_decode_bf16",
                             [_P, _P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_int, c_int, c_int, _P, _P, _P])


def attention_decode_supported(dtype, head_dim):
    return dtype == torch.bfloat16 and head_dim % 32 == 0 and 32 <= head_dim <= MAX_HEAD_DIM


def attention_decode_bf16(out, q, n_tokens, positions, token_slot, k_pages, v_pages, block_table,
                          n_q_heads, n_kv_heads, head_dim, scale, window=None, n_splits=1,
                          keys_per_split=0, part_acc=None, part_ml=None):
    """One query token per row of ``q`` (bfloat16, head_dim a multiple of 32): same contract
    as :func:`attention_generic`; ``keys_per_split`` must be a multiple of 16, or 0 to cut
    every token's own visible keys into ``n_splits`` equal parts."""
    _need_cuda(out, q, positions, token_slot, k_pages, v_pages, block_table, part_acc, part_ml)
    _need(attention_decode_supported(q.dtype, head_dim),
          "attention_decode_bf16: bfloat16 and a head size that is a multiple of 32")
    _need(out.dtype == q.dtype == k_pages.dtype, "attention: one dtype for q, cache and out")
    _need(out.is_contiguous() and out.shape[-1] == n_q_heads * head_dim, "attention: out [T, NQ*D]")
    _need(q.stride(-1) == 1 and q.stride(0) % 8 == 0, "attention: dense, 16-byte aligned q rows")
    if n_splits > 1:
        _need(keys_per_split % 16 == 0, "attention_decode_bf16: keys_per_split multiple of 16")
        _need(part_acc is not None and part_ml is not None
              and part_acc.numel() >= n_tokens * n_q_heads * n_splits * head_dim
              and part_ml.numel() >= n_tokens * n_q_heads * n_splits * 2, "attention: split buffers")
    _attention_cost(q, n_tokens, positions, n_q_heads, n_kv_heads, head_dim, window, False)
    _attn_decode_bf16(_ptr(out), _ptr(q), q.stride(0), _ptr(positions), _ptr(token_slot),
                      _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.stride(0),
                      n_tokens, n_q_heads, n_kv_heads, head_dim, float(scale), int(window or 0),
                      n_splits, keys_per_split, _ptr(part_acc), _ptr(part_ml), _stream())
    if n_splits > 1:
        count_extra_launches()               # the merge kernel


_attn_decode_tma = Function("attention_decode_tma", "ek_attention_decode_tma",
                            [_P, _P, c_int, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_int, c_int, _P, _P])
_attn_decode_tma_max = Function("attention_decode_tma", "ek_attention_decode_tma_max_splits", [c_int],
                                check_status=False)
DECODE_TMA_PORTABLE_SPLITS = 8
_decode_tma_max_splits = {}


def decode_tma_max_splits(head_dim, device=None):
    """Blocks that may share one token's pages in :func:`attention_decode_tma`: 16 where the device
    schedules thread-block clusters of that size for this head size, else the portable 8."""
    key = (head_dim, torch.cuda.current_device() if device is None else torch.device(device).index)
    if key not in _decode_tma_max_splits:
        with torch.cuda.device(key[1] if key[1] is not None else torch.cuda.current_device()):
            n = int(_attn_decode_tma_max(head_dim))
        _decode_tma_max_splits[key] = n if n in (8, 16) else DECODE_TMA_PORTABLE_SPLITS
    return _decode_tma_max_splits[key]


def attention_decode_tma_supported(dtype, head_dim, n_q_heads, n_kv_heads):
    return dtype == torch.bfloat16 and head_dim in (64, 128) and n_q_heads // n_kv_heads <= 16


def attention_decode_tma(out, q, n_tokens, positions, token_slot, k_pages, v_pages, block_table,
                         n_q_heads, n_kv_heads, head_dim, scale, window=None, n_splits=1):
    """One new token per sequence (bfloat16, head size 64 or 128, at most 16 heads a group): the
    cache pages come by TMA, started before the kernel ahead has finished; ``n_splits`` (1 to 8)
    blocks (16 where :func:`decode_tma_max_splits` says so) share a token's pages and merge inside
    a thread-block cluster.

    Precondition: ``positions``, ``token_slot`` and ``block_table`` are read before the kernel
    waits for the one ahead of it, so whatever wrote them (an upload, the state advance of the
    step before) must be separated from this launch by a launch that is not programmatic:
    :func:`embed`, the first kernel of every step, is one."""
    _need_cuda(out, q, positions, token_slot, k_pages, v_pages, block_table)
    _need(attention_decode_tma_supported(q.dtype, head_dim, n_q_heads, n_kv_heads),
          "attention_decode_tma: bfloat16, head size 64 or 128, at most 16 query heads a KV head")
    _need(out.dtype == q.dtype == k_pages.dtype, "attention: one dtype for q, cache and out")
    _need(out.is_contiguous() and out.shape[-1] == n_q_heads * head_dim, "attention: out [T, NQ*D]")
    _need(q.stride(-1) == 1 and q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0,
          "attention: dense, 4-byte aligned q rows")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim), "attention: pages [P, NKV, 64, D]")
    _need(1 <= n_splits <= decode_tma_max_splits(head_dim, q.device),
          f"attention_decode_tma: 1 to {decode_tma_max_splits(head_dim, q.device)} splits on this device")
    _need(n_tokens <= 65535, "attention_decode_tma: at most 65535 tokens a call")
    _attention_cost(q, n_tokens, positions, n_q_heads, n_kv_heads, head_dim, window, False)
    _attn_decode_tma(_ptr(out), _ptr(q), q.stride(0), _ptr(positions), _ptr(token_slot),
                     _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table),
                     block_table.stride(0), n_tokens, n_q_heads, n_kv_heads, head_dim, float(scale),
                     int(window or 0), n_splits, _ptr(tc_status(q.device)), _stream())


_attn_prefill_bf16 = Function("attention_prefill_bf16", "ek_attention_prefill_bf16",
                              [_P, _P, c_int, _P, _P, _P, c_int, c_int, _P, _P, _P, c_int, c_int,
                               c_int, c_int, c_float, c_int, _P])


def attention_prefill_supported(dtype, head_dim, n_q_heads, n_kv_heads):
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= MAX_HEAD_DIM
            and n_q_heads // n_kv_heads <= 128)


def attention_prefill_bf16(out, q, n_tokens, positions, token_slot, cu_seqlens, n_seqs, k_pages,
                           v_pages, block_table, n_q_heads, n_kv_heads, head_dim, scale,
                           window=None):
    """Several new tokens per sequence (bfloat16): sequence b owns rows cu_seqlens[b] ..
    cu_seqlens[b+1] of ``q``, which stand at consecutive positions; their keys and values
    are already in the pages."""
    _need_cuda(out, q, positions, token_slot, cu_seqlens, k_pages, v_pages, block_table)
    _need(attention_prefill_supported(q.dtype, head_dim, n_q_heads, n_kv_heads),
          "attention_prefill_bf16: bfloat16, head size a multiple of 16, at most 128 heads a group")
    _need(out.dtype == q.dtype == k_pages.dtype, "attention: one dtype for q, cache and out")
    _need(out.is_contiguous() and out.shape[-1] == n_q_heads * head_dim, "attention: out [T, NQ*D]")
    _need(q.stride(-1) == 1 and q.stride(0) % 8 == 0, "attention: dense, 16-byte aligned q rows")
    _need(cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1, "attention: cu_seqlens")
    _attention_cost(q, n_tokens, positions, n_q_heads, n_kv_heads, head_dim, window, True)
    _attn_prefill_bf16(_ptr(out), _ptr(q), q.stride(0), _ptr(positions), _ptr(token_slot),
                       _ptr(cu_seqlens), n_seqs, n_tokens, _ptr(k_pages), _ptr(v_pages),
                       _ptr(block_table), block_table.stride(0), n_q_heads, n_kv_heads, head_dim,
                       float(scale), int(window or 0), _stream())


_attn_prefill_tc = Function("attention_prefill_tc", "ek_attention_prefill_tc",
                            [_P, _P, c_int, _P, c_int, c_int, _P, _P, c_int, _P, c_int, c_int,
                             c_int, c_int, c_float, c_int, _P, _P])
_attn_prefill_tiles = Function("attention_prefill_tc", "ek_attention_prefill_tiles",
                               [_P, c_int, _P, _P, _P, c_int, c_int, c_int, _P])
PREFILL_TC_ROWS = 128       # (token, query head of a group) rows a block of attention_prefill_tc owns
PREFILL_TC_MAX_SEQS = 1024


def attention_prefill_tc_supported(dtype, head_dim, n_q_heads, n_kv_heads):
    group = n_q_heads // n_kv_heads
    return dtype == torch.bfloat16 and head_dim in (64, 128) and 128 % group == 0


_l2_bytes = {}
PREFILL_BAND_L2_SHARE = 0.5


def prefill_band_tokens(n_kv_heads, head_dim, device=None) -> int:
    """Tokens of context whose 16-bit keys and values of one layer fill ``PREFILL_BAND_L2_SHARE`` of
    the device's L2: the sequences that the prompt attention works on together."""
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None \
        else torch.device(device).index
    if index not in _l2_bytes:
        _l2_bytes[index] = int(torch.cuda.get_device_properties(index).L2_cache_size)
    return max(1, int(_l2_bytes[index] * PREFILL_BAND_L2_SHARE) // (4 * n_kv_heads * head_dim))


def attention_prefill_tiles(tiles, n_tokens, positions, token_slot, cu_seqlens, n_seqs, n_q_heads, n_kv_heads,
                            head_dim):
    """Fill ``tiles`` (int32 [>= tiles_needed, 4]) with the table of tiles that
    :func:`attention_prefill_tc` walks for this step's sequences and these head counts: (first token,
    tokens, position of the first, slot) per tile; the sequences in bands whose keys and values fit
    L2 together (longest context first), inside a band the longest key ranges first; padded with
    empty tiles.
    It is read by the attention kernels before they wait for the kernel ahead of them, so it has
    to be made before the step's first kernel (:func:`embed`, a plain launch), not just before the
    attention; returns the number of entries to pass on."""
    _need_cuda(tiles, positions, token_slot, cu_seqlens)
    tok_per_tile = PREFILL_TC_ROWS // (n_q_heads // n_kv_heads)
    need = -(-n_tokens // tok_per_tile) + n_seqs
    _need(tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.numel() >= 4 * need
          and tiles.data_ptr() % 16 == 0, "attention_prefill_tiles: int32 [tiles, 4], 16-byte aligned")
    _need(n_seqs <= PREFILL_TC_MAX_SEQS, f"attention_prefill_tc: at most {PREFILL_TC_MAX_SEQS} sequences a step")
    _need(cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1, "attention: cu_seqlens")
    _attn_prefill_tiles(_ptr(tiles), need, _ptr(cu_seqlens), _ptr(positions), _ptr(token_slot), n_seqs,
                        tok_per_tile, prefill_band_tokens(n_kv_heads, head_dim, tiles.device), _stream())
    return need


def attention_prefill_tc(out, q, n_tokens, positions, token_slot, cu_seqlens, n_seqs, k_pages,
                         v_pages, block_table, n_q_heads, n_kv_heads, head_dim, scale, window=None,
                         tiles=None, n_tiles=0):
    """:func:`attention_prefill_bf16` on tcgen05 tensor cores (head sizes 64 and 128, groups
    that divide 128): TMA-fed pages, scores and P.V in TMEM.  ``tiles`` / ``n_tiles``: the table
    :func:`attention_prefill_tiles` made for this step (made once, before the step's first
    kernel, and used by every layer); without it the table is made here and the stream is
    waited for, which suits a single call, not a model's step."""
    _need_cuda(out, q, positions, token_slot, cu_seqlens, k_pages, v_pages, block_table, tiles)
    _need(attention_prefill_tc_supported(q.dtype, head_dim, n_q_heads, n_kv_heads),
          "attention_prefill_tc: bfloat16, head size 64 or 128, a group size that divides 128")
    _need(out.dtype == q.dtype == k_pages.dtype, "attention: one dtype for q, cache and out")
    _need(out.is_contiguous() and out.shape[-1] == n_q_heads * head_dim, "attention: out [T, NQ*D]")
    _need(q.stride(-1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0,
          "attention: dense, 16-byte aligned q rows")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim), "attention: pages [P, NKV, 64, D]")
    if tiles is None:
        tok_per_tile = PREFILL_TC_ROWS // (n_q_heads // n_kv_heads)
        tiles = torch.empty((-(-n_tokens // tok_per_tile) + n_seqs, 4), dtype=torch.int32, device=q.device)
        n_tiles = attention_prefill_tiles(tiles, n_tokens, positions, token_slot, cu_seqlens, n_seqs,
                                          n_q_heads, n_kv_heads, head_dim)
        torch.cuda.current_stream().synchronize()
    _need(tiles.dtype == torch.int32 and tiles.numel() >= 4 * n_tiles and tiles.data_ptr() % 16 == 0,
          "attention_prefill_tc: the table of tiles")
    _attention_cost(q, n_tokens, positions, n_q_heads, n_kv_heads, head_dim, window, True)
    _attn_prefill_tc(_ptr(out), _ptr(q), q.stride(0), _ptr(tiles), n_tiles, n_tokens, _ptr(k_pages),
                     _ptr(v_pages), k_pages.shape[0], _ptr(block_table), block_table.stride(0), n_q_heads,
                     n_kv_heads, head_dim, float(scale), int(window or 0),
                     _ptr(tc_status(q.device)), _stream())


# ------------------------------------------------------------------ matrix products
_gemm_f32 = Function("gemm_f32", "ek_gemm_nt_f32",
                     [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P])
EPI_BF16, EPI_F32, EPI_SWIGLU = 0, 1, 2


def gemm_f32(out, x, w, n_rows=None):
    """out[M, N] = x[M, K] . w[N, K]^T in true 32-bit."""
    _need_cuda(out, x, w)
    _need(out.dtype == x.dtype == w.dtype == torch.float32, "gemm_f32: float32 tensors")
    _need(x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1, "gemm_f32: dense rows")
    m = n_rows if n_rows is not None else x.shape[0]
    n, k = w.shape
    _need(x.shape[-1] == k and out.shape[-1] == n and out.shape[0] >= m, "gemm_f32: shapes disagree")
    if lib.recording():
        lib.annotate(bytes=4 * (n * k + m * k + m * n), flops=2 * m * n * k)
    _gemm_f32(_ptr(out), _ptr(x), _ptr(w), m, n, k, x.stride(0), w.stride(0), out.stride(0), _stream())


B200_SM_COUNT = 148        # used only where no device can be asked (launch plans worked out on a CPU box)
_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current one if None), asked once."""
    if not torch.cuda.is_available():
        return B200_SM_COUNT
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None \
        else torch.device(device).index
    if index not in _sm_counts:
        _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _sm_counts[index]


_SPLIT_PARTIAL_FLOATS = 4 * 1024 * 1024      # 16 MiB of split partials per device
_SPLIT_TICKETS = 16384
_split_scratch = {}


def split_scratch(device):
    """Per-device scratch of products whose K is split over more blocks than a cluster holds:
    partial tiles and zeroed tickets.  Created on first use; create it before capturing a graph
    (``ModelRunner`` does)."""
    key = str(torch.device(device))
    if key not in _split_scratch:
        _split_scratch[key] = (torch.empty(_SPLIT_PARTIAL_FLOATS, dtype=torch.float32, device=device),
                               torch.zeros(_SPLIT_TICKETS, dtype=torch.int32, device=device))
    return _split_scratch[key]


_gemm_tc = Function("gemm_tc_bf16", "ek_gemm_tc_bf16",
                    [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     _P, _P, c_longlong, c_int, _P, c_int, c_int, c_float, _P, c_int, _P, _P, _P, _P])
_tc_status = {}
TC_SWAP_MAX_ROWS = 64


def tc_status(device):
    """One int per device that the tensor-core GEMM sets when a barrier wait times out."""
    key = str(torch.device(device))
    if key not in _tc_status:
        _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[key]


def check_tc_status(device):
    """Synchronises; raises if a kernel gave up a bounded barrier wait since the last check (products:
    1 producer, 2 MMA, 3 epilogue, 4 copies before exit; decode attention 41, 42; others by their
    kernel) and clears the word, so that the next check speaks of later launches only."""
    code = int(tc_status(device).item())
    if code:
        tc_status(device).zero_()
        raise KernelError(f"a bounded barrier wait ran out in a tensor-core kernel (code {code}); "
                          "results since the last check are invalid")


_wait_that_runs_out = Function("gemm_tc_bf16", "ek_tc_wait_that_runs_out", [_P, c_int, ctypes.c_uint, _P])


def wait_that_runs_out(device, code=77, limit=4096):
    """Launch one thread that waits ``limit`` rounds for a barrier nothing completes, gives up and
    records ``code`` in the device's status word - what a kernel does when a wait of its own runs
    out.  The kernel ends by itself; :func:`check_tc_status` then raises."""
    with torch.cuda.device(device):
        _wait_that_runs_out(_ptr(tc_status(device)), int(code), int(limit), _stream())


TC_MAX_CLUSTER = 8          # blocks of a thread-block cluster (the portable limit)


def swap_k_split(n_out, k, epilogue):
    """Blocks that share a tile's K in the swapped form: two blocks fit an SM - fill those 296
    places, keep at least 8 K blocks a block, stay within one cluster, and take a power of two
    (clusters of 3, 5, 6 or 7 blocks do not pack the GPCs evenly: 5 -> 4 was worth 0.6-1 % of a step)."""
    tiles = -(-n_out // (64 if epilogue == EPI_SWIGLU else 128))
    k_blocks = -(-k // 64)
    split = max(1, min(2 * sm_count() // tiles, k_blocks // 8, TC_MAX_CLUSTER))
    return 1 << (split.bit_length() - 1)


def gemm_tc_bf16(out, x, w, epilogue=EPI_BF16, n_rows=None, swap=None, k_split=None, cluster=True,
                 row_scale=None, residual=None):
    """out = x . w^T (or the SwiGLU of it) on tcgen05 tensor cores with TMA-staged operands.

    ``swap`` (default: at most 64 rows) puts the weights on the 128-row side of the MMA and
    splits K over ``k_split`` blocks; otherwise 128 x 128 tiles of the output.  Up to 8 splits
    add their partial tiles through the distributed shared memory of a thread-block cluster
    (``cluster``), more of them through scratch in global memory.

    Two options of the swapped form carry a norm that was moved out of its own kernel.
    ``row_scale=(ss, size, eps)``: row r of the 32-bit result is multiplied by
    rsqrt(sum(ss[r, :]) / size + eps) before the epilogue (``ss`` [rows, tiles], 32-bit).
    ``residual=(stream, gain, ss_out)`` (bfloat16 result, N a multiple of 4): the result is added to
    the 32-bit ``stream`` [rows, N] in place, ``out`` gets stream * gain, and ``ss_out`` [rows,
    ceil(N / 128)] the sum of stream^2 over each 128-column tile.
    """
    _need_cuda(out, x, w)
    m = n_rows if n_rows is not None else x.shape[0]
    n, k = w.shape
    _need(x.dtype == w.dtype == torch.bfloat16, "gemm_tc_bf16: bfloat16 operands")
    _need(k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0,
          f"gemm_tc_bf16: inner size {k} and row strides must be multiples of 8")
    _need(x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1 and x.shape[-1] == k,
          "gemm_tc_bf16: dense rows of matching inner size")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemm_tc_bf16: 16-byte aligned operands")
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    _need(out.shape[-1] == n_out and out.shape[0] >= m, "gemm_tc_bf16: out shape")
    _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "gemm_tc_bf16: out dtype")
    if swap is None:
        swap = m <= TC_SWAP_MAX_ROWS
    _need(not swap or m <= TC_SWAP_MAX_ROWS, "gemm_tc_bf16: the swapped form takes at most 64 rows")
    partials, tickets = split_scratch(x.device)
    if k_split is None:
        k_split = swap_k_split(n_out, k, epilogue) if swap else 1
    if row_scale is not None or residual is not None:
        cluster, k_split = True, min(k_split, TC_MAX_CLUSTER)     # these forms have no scratch path
    ss_in, ss_tiles, size, eps = None, 0, 0, 0.0
    if row_scale is not None:
        ss_in, size, eps = row_scale
        _need(swap and ss_in.dtype == torch.float32 and ss_in.is_contiguous() and ss_in.dim() == 2
              and ss_in.shape[0] >= m and ss_in.is_cuda, "gemm_tc_bf16: row_scale needs 32-bit sums [rows, tiles]")
        ss_tiles = ss_in.shape[1]
    stream, gain, ss_out, ld_stream = None, None, None, 0
    if residual is not None:
        stream, gain, ss_out = residual
        _need_cuda(stream, gain, ss_out)
        _need(swap and epilogue == EPI_BF16 and n % 4 == 0 and out.stride(0) % 4 == 0,
              "gemm_tc_bf16: residual needs the swapped form, a bfloat16 result and N a multiple of 4")
        _need(stream.dtype == torch.float32 and stream.stride(-1) == 1 and stream.stride(0) % 4 == 0
              and stream.shape[-1] == n and stream.shape[0] >= m and stream.data_ptr() % 16 == 0,
              "gemm_tc_bf16: residual stream [rows, N] in 32-bit, 16-byte aligned rows")
        _need(gain.dtype == torch.float32 and gain.numel() == n and gain.data_ptr() % 16 == 0,
              "gemm_tc_bf16: gain [N] in 32-bit")
        _need(ss_out.dtype == torch.float32 and ss_out.is_contiguous() and ss_out.shape[0] >= m
              and ss_out.shape[1] == -(-n // 128), "gemm_tc_bf16: ss_out [rows, ceil(N/128)] in 32-bit")
        ld_stream = stream.stride(0)
    if lib.recording():
        moved = 2 * (n * k + m * k) + m * n_out * out.element_size() + (8 * m * n if residual is not None else 0)
        lib.annotate(bytes=moved, flops=2 * m * n * k, label=f"{n}x{k}")
    _gemm_tc(_ptr(out), _ptr(x), _ptr(w), m, n, k, x.stride(0), w.stride(0), out.stride(0),
             epilogue, 1 if swap else 0, k_split, 1 if cluster else 0, _ptr(partials), _ptr(tickets),
             _SPLIT_PARTIAL_FLOATS, _SPLIT_TICKETS, _ptr(ss_in), ss_tiles, int(size), float(eps),
             _ptr(stream), ld_stream, _ptr(gain), _ptr(ss_out), _ptr(tc_status(x.device)), _stream())


_gemm_pair = Function("gemm_pair_bf16", "ek_gemm_pair_bf16",
                      [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P])
PAIR_EPI_BF16, PAIR_EPI_ADD_F32, PAIR_EPI_SWIGLU = 0, 1, 2


def gemm_pair_takes(out, x, w, epilogue) -> bool:
    """Whether :func:`gemm_pair_bf16` can address these operands (16-byte aligned rows)."""
    return (x.dtype == w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and out.stride(0) % (4 if epilogue == PAIR_EPI_ADD_F32 else 8) == 0)


def gemm_pair_bf16(out, x, w, epilogue=PAIR_EPI_BF16, n_rows=None):
    """The product for many rows on pairs of SMs (``tcgen05.mma.cta_group::2``, 256 x 256 tiles, a
    persistent launch).  ``PAIR_EPI_BF16``: out [M, N] = x . w^T in bfloat16; ``PAIR_EPI_ADD_F32``:
    out [M, N] (32-bit) += x . w^T; ``PAIR_EPI_SWIGLU``: out [M, N / 2] = silu(x . wg^T) * (x . wu^T)
    with w = [gate rows; up rows]."""
    _need_cuda(out, x, w)
    m = n_rows if n_rows is not None else x.shape[0]
    n, k = w.shape
    _need(gemm_pair_takes(out, x, w, epilogue) and x.shape[-1] == k,
          "gemm_pair_bf16: bfloat16 operands with dense, 16-byte aligned rows of matching inner size")
    _need(epilogue in (PAIR_EPI_BF16, PAIR_EPI_ADD_F32, PAIR_EPI_SWIGLU), "gemm_pair_bf16: epilogue")
    _need(epilogue != PAIR_EPI_SWIGLU or n % 2 == 0, "gemm_pair_bf16: SwiGLU needs gate and up rows")
    n_out = n // 2 if epilogue == PAIR_EPI_SWIGLU else n
    _need(out.shape[-1] == n_out and out.shape[0] >= m and x.shape[0] >= m, "gemm_pair_bf16: out shape")
    _need(out.dtype == (torch.float32 if epilogue == PAIR_EPI_ADD_F32 else torch.bfloat16),
          "gemm_pair_bf16: out dtype")
    if lib.recording():
        moved = 2 * (n * k + m * k) + m * n_out * (8 if epilogue == PAIR_EPI_ADD_F32 else 2)
        lib.annotate(bytes=moved, flops=2 * m * n * k, label=f"{n}x{k}")
    _gemm_pair(_ptr(out), _ptr(x), _ptr(w), m, n, k, x.stride(0), w.stride(0), out.stride(0), epilogue,
               _ptr(tc_status(x.device)), _stream())


_gemm_tc_qkv = Function("gemm_tc_bf16", "ek_gemm_tc_qkv_rope",
                        [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int, c_int, c_float,
                         _P, _P, c_float, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P])
QKV_ROPE_HEAD_DIM = 128


def gemm_tc_qkv_rope(qkv, x, w, n_rows, q_gain, k_gain, qk_eps, cos, sin, positions, token_slot, k_pages,
                     v_pages, block_table, n_q_heads, n_kv_heads, write_kv=True, row_scale=None,
                     k_split=None):
    """The q/k/v product of an attention layer with heads of 128, fully rotated, for at most 64
    rows, with :func:`qk_norm_rope_kv` done in its epilogue on the 32-bit sums: q (normalised,
    rotated) goes to the q part of ``qkv`` [rows, (NQ + 2 NKV) * 128], k and v to the pages.
    ``row_scale`` as in :func:`gemm_tc_bf16`."""
    _need_cuda(qkv, x, w, cos, sin, positions, token_slot, k_pages, v_pages, block_table)
    m, (n, k) = n_rows, w.shape
    _need(x.dtype == w.dtype == qkv.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16,
          "gemm_tc_qkv_rope: bfloat16 operands, result and cache")
    _need(m <= TC_SWAP_MAX_ROWS and n == (n_q_heads + 2 * n_kv_heads) * QKV_ROPE_HEAD_DIM,
          "gemm_tc_qkv_rope: at most 64 rows, heads of 128")
    _need(k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(-1) == 1
          and w.stride(-1) == 1 and x.shape[-1] == k and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0,
          "gemm_tc_qkv_rope: dense, 16-byte aligned operand rows")
    _need(qkv.stride(-1) == 1 and qkv.shape[-1] == n and qkv.stride(0) % 4 == 0 and qkv.shape[0] >= m,
          "gemm_tc_qkv_rope: qkv [rows, (NQ + 2 NKV) * 128]")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
          and sin.is_contiguous() and cos.shape[-1] == QKV_ROPE_HEAD_DIM // 2,
          "gemm_tc_qkv_rope: 32-bit tables of 64 columns")
    for g in (q_gain, k_gain):
        _need(g is None or (g.is_cuda and g.dtype == torch.float32 and g.numel() == QKV_ROPE_HEAD_DIM),
              "qk gains: 32-bit [128]")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and k_pages.shape[1:] == (n_kv_heads, PAGE, QKV_ROPE_HEAD_DIM), "attention: pages [P, NKV, 64, 128]")
    _need(block_table.dtype == torch.int32 and positions.dtype == torch.int32
          and token_slot.dtype == torch.int32, "gemm_tc_qkv_rope: int32 indices")
    ss_in, ss_tiles, size, eps = None, 0, 0, 0.0
    if row_scale is not None:
        ss_in, size, eps = row_scale
        _need(ss_in.is_cuda and ss_in.dtype == torch.float32 and ss_in.is_contiguous() and ss_in.dim() == 2
              and ss_in.shape[0] >= m, "gemm_tc_qkv_rope: row_scale needs 32-bit sums [rows, tiles]")
        ss_tiles = ss_in.shape[1]
    if k_split is None:
        k_split = swap_k_split(n, k, EPI_BF16)
    if lib.recording():
        lib.annotate(bytes=2 * (n * k + m * k + m * n), flops=2 * m * n * k)
    _gemm_tc_qkv(_ptr(qkv), _ptr(x), _ptr(w), m, k, x.stride(0), w.stride(0), qkv.stride(0), k_split,
                 _ptr(ss_in), ss_tiles, int(size), float(eps), _ptr(q_gain), _ptr(k_gain), float(qk_eps),
                 _ptr(cos), _ptr(sin), _ptr(positions), _ptr(token_slot), _ptr(k_pages), _ptr(v_pages),
                 _ptr(block_table), block_table.stride(0), n_q_heads, n_kv_heads, 1 if write_kv else 0,
                 _ptr(tc_status(x.device)), _stream())


_gemm_pair_qkv = Function("gemm_pair_bf16", "ek_gemm_pair_qkv_rope",
                          [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, c_float, _P, _P, _P, _P, _P,
                           _P, _P, c_int, c_int, c_int, c_int, _P, _P])


def gemm_pair_qkv_rope(qkv, x, w, n_rows, q_gain, k_gain, qk_eps, cos, sin, positions, token_slot, k_pages,
                       v_pages, block_table, n_q_heads, n_kv_heads, write_kv=True):
    """The q/k/v product of many rows (the pair kernel) with the per-head RMSNorm of q and k, the rotation
    and the cache write in its epilogue (heads of 128, fully rotated).  Of ``qkv`` only the q columns are
    written; k and v go to the pages.  Rows with a negative position are skipped."""
    _need_cuda(qkv, x, w, cos, sin, positions, token_slot, k_pages, v_pages, block_table)
    m, (n, k) = n_rows, w.shape
    _need(x.dtype == w.dtype == qkv.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16,
          "gemm_pair_qkv_rope: bfloat16 operands, result and cache")
    _need(n == (n_q_heads + 2 * n_kv_heads) * QKV_ROPE_HEAD_DIM and gemm_pair_takes(qkv, x, w, PAIR_EPI_BF16)
          and x.shape[-1] == k and x.shape[0] >= m,
          "gemm_pair_qkv_rope: heads of 128, dense 16-byte aligned operand rows")
    _need(qkv.shape[-1] == n and qkv.shape[0] >= m, "gemm_pair_qkv_rope: qkv [rows, (NQ + 2 NKV) * 128]")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous()
          and sin.is_contiguous() and cos.shape[-1] == QKV_ROPE_HEAD_DIM // 2,
          "gemm_pair_qkv_rope: 32-bit tables of 64 columns")
    for g in (q_gain, k_gain):
        _need(g is None or (g.is_cuda and g.dtype == torch.float32 and g.numel() == QKV_ROPE_HEAD_DIM),
              "qk gains: 32-bit [128]")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dim() == 4
          and k_pages.shape[1:] == (n_kv_heads, PAGE, QKV_ROPE_HEAD_DIM), "attention: pages [P, NKV, 64, 128]")
    _need(block_table.dtype == torch.int32 and positions.dtype == torch.int32
          and token_slot.dtype == torch.int32 and positions.numel() >= m and token_slot.numel() >= m,
          "gemm_pair_qkv_rope: int32 indices, one per row")
    if lib.recording():
        lib.annotate(bytes=2 * (n * k + m * k + m * n), flops=2 * m * n * k, label=f"{n}x{k}")
    _gemm_pair_qkv(_ptr(qkv), _ptr(x), _ptr(w), m, k, x.stride(0), w.stride(0), qkv.stride(0),
                   _ptr(q_gain), _ptr(k_gain), float(qk_eps), _ptr(cos), _ptr(sin), _ptr(positions),
                   _ptr(token_slot), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.stride(0),
                   n_q_heads, n_kv_heads, 1 if write_kv else 0, _ptr(tc_status(x.device)), _stream())


# ------------------------------------------------------------------ sampling and decode state
_sample = Function("sampling", "ek_sample",
                   [_P, _P, c_longlong, c_int, c_int, c_float, c_int, c_ulonglong, _P, _P, _P, _P, _P])
_sample_wide = Function("sampling", "ek_sample_wide",
                        [_P, _P, c_longlong, c_int, c_int, c_float, c_ulonglong, _P, _P, _P, _P, _P,
                         _P, c_int, _P])
_decode_advance = Function("sampling", "ek_decode_advance",
                           [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P])


def sampling_settings(temperature, top_k, seed, device):
    """The 4-int device block ``sample(dyn=...)`` reads its settings from."""
    import struct
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    bits = struct.unpack("<i", struct.pack("<f", float(temperature)))[0]
    lo, hi = seed & 0xFFFFFFFF, seed >> 32
    as_i32 = lambda v: v - (1 << 32) if v >= (1 << 31) else v
    return torch.tensor([bits, int(top_k), as_i32(lo), as_i32(hi)], dtype=torch.int32, device=device)


def sample(out_token, logits, temperature, top_k, seed, streams=None, draws=None, active=None,
           n_rows=None, dyn=None):
    """out_token[r] from logits[r, :] (32-bit): arg-max when temperature is 0, else
    Gumbel-max over the top_k largest (0: all).  ``dyn`` (see ``sampling_settings``)
    overrides temperature, top_k and seed from device memory."""
    _need_cuda(out_token, logits, streams, draws, active, dyn)
    _need(logits.dtype == torch.float32 and logits.stride(-1) == 1, "sample: dense 32-bit logits")
    _need(out_token.dtype == torch.int32, "sample: int32 out")
    rows = n_rows if n_rows is not None else logits.shape[0]
    if lib.recording():
        lib.annotate(bytes=4 * rows * logits.shape[-1])
    _sample(_ptr(out_token), _ptr(logits), logits.stride(0), rows, logits.shape[-1],
            float(temperature), int(top_k), int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(streams),
            _ptr(draws), _ptr(active), _ptr(dyn), _stream())


SAMPLE_SEGMENTS = 32


_sample_cluster = Function("sampling", "ek_sample_cluster",
                           [_P, _P, c_longlong, c_int, c_int, c_float, c_int, c_ulonglong, _P, _P, _P, _P, _P])


def sample_cluster(out_token, logits, temperature, top_k, seed, streams=None, draws=None, active=None,
                   n_rows=None, dyn=None):
    """:func:`sample` with each row spread over the 8 blocks of a thread-block cluster (wide
    vocabularies with top-k: the radix digits are counted by all 8 and read through distributed
    shared memory).  Same tokens as :func:`sample`."""
    _need_cuda(out_token, logits, streams, draws, active, dyn)
    _need(logits.dtype == torch.float32 and logits.stride(-1) == 1, "sample: dense 32-bit logits")
    _need(out_token.dtype == torch.int32, "sample: int32 out")
    rows = n_rows if n_rows is not None else logits.shape[0]
    if lib.recording():
        lib.annotate(bytes=4 * rows * logits.shape[-1])
    _sample_cluster(_ptr(out_token), _ptr(logits), logits.stride(0), rows, logits.shape[-1],
                    float(temperature), int(top_k), int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(streams),
                    _ptr(draws), _ptr(active), _ptr(dyn), _stream())


def sample_wide(out_token, logits, temperature, seed, part_score, part_index, streams=None,
                draws=None, active=None, n_rows=None, dyn=None):
    """:func:`sample` without top-k, spread over ``SAMPLE_SEGMENTS`` blocks a row (for wide
    vocabularies).  ``part_score`` float32 / ``part_index`` int32: rows * SAMPLE_SEGMENTS each."""
    _need_cuda(out_token, logits, streams, draws, active, dyn, part_score, part_index)
    _need(logits.dtype == torch.float32 and logits.stride(-1) == 1, "sample: dense 32-bit logits")
    rows = n_rows if n_rows is not None else logits.shape[0]
    _need(part_score.dtype == torch.float32 and part_index.dtype == torch.int32
          and part_score.numel() >= rows * SAMPLE_SEGMENTS
          and part_index.numel() >= rows * SAMPLE_SEGMENTS, "sample_wide: partial buffers")
    if lib.recording():
        lib.annotate(bytes=4 * rows * logits.shape[-1])
    _sample_wide(_ptr(out_token), _ptr(logits), logits.stride(0), rows, logits.shape[-1],
                 float(temperature), int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(streams), _ptr(draws),
                 _ptr(active), _ptr(dyn), _ptr(part_score), _ptr(part_index), SAMPLE_SEGMENTS,
                 _stream())
    count_extra_launches()                   # partial kernel + final kernel


def decode_advance(sampled, token_ids, positions, draws, remaining, out_tokens, step_index,
                   stop_ids, n_stop, batch):
    _need_cuda(sampled, token_ids, positions, draws, remaining, out_tokens, step_index, stop_ids)
    for t in (sampled, token_ids, positions, draws, remaining, out_tokens, step_index):
        _need(t.dtype == torch.int32, "decode_advance: int32 state")
    _need(out_tokens.shape[-1] == batch, "decode_advance: out_tokens [steps, batch]")
    _decode_advance(_ptr(sampled), _ptr(token_ids), _ptr(positions), _ptr(draws), _ptr(remaining),
                    _ptr(out_tokens), _ptr(step_index), _ptr(stop_ids), n_stop, batch,
                    out_tokens.shape[0], _stream())


def build_all():
    """Compile every kernel library (used by the build check)."""
    from . import build
    return build.build_all()
