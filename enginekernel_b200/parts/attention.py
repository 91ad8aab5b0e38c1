"""Grouped-query attention over the paged cache.

Per token: q/k/v projections without bias (one fused product), optional RMSNorm of each
query and key head over the head dimension, position encoding of queries and keys, keys
and values stored in the cache entry, softmax(scale * q.K^T) V over the keys the token may
see (all earlier ones, or the last ``window``), output projection
(engine/ek_model.py:298-325 for prompts, 380-403 for decode; formula 475-488).
Query head h reads KV head h // (num_heads // num_kv_heads).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``,
``qk_norm_eps`` (None: no q/k norm), ``window`` (None: all keys), ``position`` (a
position PartSpec or None).  Tensors: ``q`` [NH*D, H], ``k``, ``v`` [NKV*D, H], ``o``
[H, NH*D], and with q/k norm ``q_norm``, ``k_norm`` [D].  q, k and v are concatenated at
load as the reference does (engine/ek_model.py:140-144).
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear, pair_product_wins, row_scale_of, tc_takes
from ..registry import lookup_part, register_part
from .base import DeferredNorm, Mixer
from .spec import CacheSpec, TensorSpec

FUSE_ROPE_ROWS = 64       # the q/k/v product does norm, rotation and cache write itself up to here
WIDE_CLUSTER_PAGES = 64     # clusters of more than 8 key splits only from this many pages of context


@register_part("mixer", "attention")
class Attention(Mixer):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, nh, nkv, d = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"]
        out = [TensorSpec(w["q"], (nh * d, h)), TensorSpec(w["k"], (nkv * d, h)),
               TensorSpec(w["v"], (nkv * d, h)), TensorSpec(w["o"], (h, nh * d))]
        if p.get("qk_norm_eps") is not None:
            out += [TensorSpec(w["q_norm"], (d,), "gain"), TensorSpec(w["k_norm"], (d,), "gain")]
        return out

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(self.param("hidden_size"))
        self.num_heads = int(self.param("num_heads"))
        self.num_kv_heads = int(self.param("num_kv_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.scale = float(self.param("scale"))
        self.qk_norm_eps = spec.params.get("qk_norm_eps")
        self.window = spec.params.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        kernels.check_head_dim(self.head_dim)
        pos = spec.params.get("position")
        self.position = lookup_part("position", pos.kind)(pos, dtype, device) if pos else None
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    def cache_spec(self):
        return CacheSpec("kv", heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window)

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def _tiles_key(self):
        return ("prefill_tc_tiles", self.num_heads // self.num_kv_heads, self.num_kv_heads * self.head_dim)

    def begin_step(self, ctx):
        """The table of tiles of the tcgen05 prompt attention, once per step and shape of the heads."""
        if ctx.is_decode or ctx.n_seqs > kernels.PREFILL_TC_MAX_SEQS or not kernels.attention_prefill_tc_supported(
                self.dtype, self.head_dim, self.num_heads, self.num_kv_heads):
            return
        key = self._tiles_key()
        if key in ctx.shared:
            return
        per_tile = kernels.PREFILL_TC_ROWS // (self.num_heads // self.num_kv_heads)
        rows = -(-ctx.n_tokens // per_tile) + ctx.n_seqs
        tiles = ctx.workspace.get(f"prefill_tc_tiles_{key[1]}_{key[2]}", (rows, 4), torch.int32)
        n = kernels.attention_prefill_tiles(tiles, ctx.n_tokens, ctx.positions, ctx.token_slot, ctx.cu_seqlens,
                                            ctx.n_seqs, self.num_heads, self.num_kv_heads, self.head_dim)
        ctx.shared[key] = (tiles, n)

    def load(self, tensors):
        w = self.spec.weights
        self.w_qkv = torch.cat([tensors[w["q"]], tensors[w["k"]], tensors[w["v"]]], dim=0) \
            .to(self.dtype).contiguous()
        self.w_o = tensors[w["o"]].to(self.dtype).contiguous()
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[w["q_norm"]].to(torch.float32).contiguous()
            self.k_gain = tensors[w["k_norm"]].to(torch.float32).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o, self.q_gain, self.k_gain)
                   if t is not None)

    # ------------------------------------------------------------------
    takes_deferred_norm = True
    defers_norm = True

    def forward(self, x, ctx, entry, writes_cache=True, defer=None):
        t = ctx.n_tokens
        pos = self.position
        if self._fuses_rope(x, ctx):
            # few rows, heads of 128: norm, rotation and cache write ride on the product's epilogue
            row_scale, xin = (row_scale_of(x), x.scaled) if isinstance(x, DeferredNorm) else (None, x)
            qkv = ctx.workspace.get("qkv", (t, self.w_qkv.shape[0]), self.dtype)
            kernels.gemm_tc_qkv_rope(
                qkv, xin, self.w_qkv, t, self.q_gain, self.k_gain,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, pos.cos, pos.sin,
                ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages, entry.block_table,
                self.num_heads, self.num_kv_heads, write_kv=writes_cache, row_scale=row_scale)
            out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
            self._attend(out, qkv, ctx, entry)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer)
        if self._fuses_rope_of_many_rows(x, ctx):
            # many rows, heads of 128: the same on the epilogue of the product on pairs of SMs
            qkv = ctx.workspace.get("qkv", (t, self.w_qkv.shape[0]), self.dtype)
            kernels.gemm_pair_qkv_rope(
                qkv, x, self.w_qkv, t, self.q_gain, self.k_gain,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, pos.cos, pos.sin,
                ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages, entry.block_table,
                self.num_heads, self.num_kv_heads, write_kv=writes_cache)
            out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
            self._attend(out, qkv, ctx, entry)
            return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer)
        qkv = linear(x, self.w_qkv, ctx, "qkv", n_rows=t)
        kernels.qk_norm_rope_kv(
            qkv, t, self.q_gain, self.k_gain,
            pos.cos if pos else _no_table(self.device), pos.sin if pos else _no_table(self.device),
            pos.rotary_dim if pos else 0, ctx.positions, ctx.token_slot, entry.k_pages,
            entry.v_pages, entry.block_table, self.num_heads, self.num_kv_heads, self.head_dim,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_kv=writes_cache)
        out = ctx.workspace.get("attn_out", (t, self.num_heads * self.head_dim), self.dtype)
        self._attend(out, qkv, ctx, entry)
        return linear(out, self.w_o, ctx, "attn_proj", n_rows=t, defer=defer)

    def _fuses_rope(self, x, ctx):
        xin = x.scaled if isinstance(x, DeferredNorm) else x
        pos = self.position
        return (self.dtype == torch.bfloat16 and ctx.n_tokens <= FUSE_ROPE_ROWS
                and self.head_dim == kernels.QKV_ROPE_HEAD_DIM and pos is not None
                and getattr(pos, "rotary_dim", 0) == self.head_dim and tc_takes(xin, self.w_qkv))

    def _fuses_rope_of_many_rows(self, x, ctx):
        pos = self.position
        if (isinstance(x, DeferredNorm) or self.dtype != torch.bfloat16
                or self.head_dim != kernels.QKV_ROPE_HEAD_DIM or pos is None
                or getattr(pos, "rotary_dim", 0) != self.head_dim):
            return False
        qkv = ctx.workspace.get("qkv", (ctx.n_tokens, self.w_qkv.shape[0]), self.dtype)
        return pair_product_wins(qkv, x, self.w_qkv, ctx.n_tokens, kernels.PAIR_EPI_BF16)

    def _attend(self, out, qkv, ctx, entry):
        t = ctx.n_tokens
        visible = min(ctx.max_context, self.window) if self.window else ctx.max_context
        fast_decode = ctx.is_decode and kernels.attention_decode_supported(self.dtype, self.head_dim)
        if not ctx.is_decode and kernels.attention_prefill_supported(
                self.dtype, self.head_dim, self.num_heads, self.num_kv_heads):
            prefill = kernels.attention_prefill_bf16
            if ctx.n_seqs <= kernels.PREFILL_TC_MAX_SEQS and kernels.attention_prefill_tc_supported(
                    self.dtype, self.head_dim, self.num_heads, self.num_kv_heads):
                prefill = kernels.attention_prefill_tc      # tcgen05: head sizes 64 and 128
            extra = {}
            if prefill is kernels.attention_prefill_tc:
                made = ctx.shared.get(self._tiles_key())
                if made is not None:                 # (made in begin_step; a part driven alone has none)
                    extra = dict(tiles=made[0], n_tiles=made[1])
            prefill(
                out, qkv, t, ctx.positions, ctx.token_slot, ctx.cu_seqlens, ctx.n_seqs,
                entry.k_pages, entry.v_pages, entry.block_table, self.num_heads, self.num_kv_heads,
                self.head_dim, self.scale, self.window, **extra)
            return
        if ctx.is_decode and t <= 65535 and kernels.attention_decode_tma_supported(
                self.dtype, self.head_dim, self.num_heads, self.num_kv_heads):
            # blocks = tokens x KV heads x splits, two fit an SM; a split takes whole pages and the
            # splits of a token are one cluster
            blocks = t * self.num_kv_heads
            pages = -(-visible // kernels.PAGE)
            # (more than 8 blocks a token only pay with many pages each: long contexts, few sequences)
            limit = kernels.decode_tma_max_splits(self.head_dim, self.device) if pages >= WIDE_CLUSTER_PAGES else \
                kernels.DECODE_TMA_PORTABLE_SPLITS
            splits = max(1, min(2 * kernels.sm_count(self.device) // blocks, pages, limit))
            splits = 1 << (splits.bit_length() - 1)      # clusters of 3, 5, 6, 7 pack the GPCs badly
            kernels.attention_decode_tma(
                out, qkv, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                entry.block_table, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                self.window, splits)
            return
        if fast_decode:
            # blocks = tokens x KV heads (x 16-row blocks of the group); three fit an SM.  Split
            # the keys so that the blocks just fill the machine once, or about twice when one
            # filling cannot be approached; never finer than two pages a split.
            blocks = t * self.num_kv_heads * -(-(self.num_heads // self.num_kv_heads) // 16)
            resident = 3 * kernels.sm_count(self.device)
            splits = resident // blocks
            if blocks * splits < 0.7 * resident:
                splits = int(1.8 * resident / blocks + 0.5)
            splits = max(1, min(splits, -(-visible // 128)))
            unit = 64
        else:
            blocks = t * self.num_heads
            splits = 1
            if blocks < 2 * kernels.sm_count(self.device) and ctx.max_context > 512:
                splits = max(1, min(-(-visible // 256), -(-4 * kernels.sm_count(self.device) // blocks), 64))
            unit = 128
        per_split, acc, ml = 0, None, None
        if splits > 1 and not fast_decode:      # the decode kernel cuts each token's own range
            per_split = -(-(-(-ctx.max_context // splits)) // unit) * unit
            splits = -(-ctx.max_context // per_split)
        if splits > 1:
            acc = ctx.workspace.get("attn_part_acc", (t, self.num_heads, splits, self.head_dim),
                                    torch.float32)
            ml = ctx.workspace.get("attn_part_ml", (t, self.num_heads, splits, 2), torch.float32)
        args = (out, qkv, t, ctx.positions, ctx.token_slot, entry.k_pages, entry.v_pages,
                entry.block_table, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                self.window, splits, per_split, acc, ml)
        fn = kernels.attention_decode_bf16 if fast_decode else kernels.attention_generic
        fn(*args)


_EMPTY = {}


def _no_table(device):
    key = str(device)
    if key not in _EMPTY:
        _EMPTY[key] = torch.zeros((1, 0), dtype=torch.float32, device=device)
    return _EMPTY[key]
