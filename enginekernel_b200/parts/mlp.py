"""Gated feed-forward (SwiGLU): down(act(gate(x)) * up(x)), no biases.

engine/ek_model.py:205-209 with engine/ek_kernels.py:125-143; gate and up are
concatenated at load (gate rows first, engine/ek_model.py:145-147).  Parameters:
``hidden_size``, ``intermediate_size``, ``activation`` ("silu").  Tensors: ``gate``,
``up`` [I, H], ``down`` [H, I].
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear, pair_product_wins, row_scale_of, tc_takes
from ..registry import register_part
from .base import DeferredNorm, FeedForward
from .spec import TensorSpec


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    @classmethod
    def tensors(cls, spec):
        p, w = spec.params, spec.weights
        h, i = p["hidden_size"], p["intermediate_size"]
        return [TensorSpec(w["gate"], (i, h)), TensorSpec(w["up"], (i, h)),
                TensorSpec(w["down"], (h, i))]

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        act = spec.params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp has no activation {act!r} (only silu)")
        self.w_gate_up = self.w_down = None

    def load(self, tensors):
        w = self.spec.weights
        self.w_gate_up = torch.cat([tensors[w["gate"]], tensors[w["up"]]], dim=0) \
            .to(self.dtype).contiguous()
        self.w_down = tensors[w["down"]].to(self.dtype).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    takes_deferred_norm = True
    defers_norm = True

    def forward(self, x, ctx, defer=None):
        t = ctx.n_tokens
        row_scale = None
        if isinstance(x, DeferredNorm):
            row_scale, x = row_scale_of(x), x.scaled
        if self.dtype == torch.bfloat16 and t <= kernels.TC_SWAP_MAX_ROWS and tc_takes(x, self.w_gate_up):
            # gate and up rows share a tile, so silu(gate) * up is formed in the epilogue
            act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
            kernels.gemm_tc_bf16(act, x, self.w_gate_up, kernels.EPI_SWIGLU, n_rows=t, swap=True,
                                 row_scale=row_scale)
        elif row_scale is not None:
            raise kernels.KernelError("a deferred norm reached a product that cannot scale its rows")
        elif self.dtype == torch.bfloat16 and pair_product_wins(
                ctx.workspace.get("mlp_act", (t, self.inter), self.dtype), x, self.w_gate_up, t,
                kernels.PAIR_EPI_SWIGLU):
            # many rows: the pair of blocks that shares a tile stages gate rows in one block and the
            # matching up rows in the other, and the epilogue forms silu(gate) * up from the 32-bit sums
            act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
            kernels.gemm_pair_bf16(act, x, self.w_gate_up, kernels.PAIR_EPI_SWIGLU, n_rows=t)
        else:
            gu = linear(x, self.w_gate_up, ctx, "mlp_gate_up", n_rows=t)
            act = ctx.workspace.get("mlp_act", (t, self.inter), self.dtype)
            kernels.silu_mul(act, gu, n_rows=t)
        return linear(act, self.w_down, ctx, "mlp_down", n_rows=t, defer=defer)
