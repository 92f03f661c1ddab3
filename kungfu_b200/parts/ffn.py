"""Gated feed-forward.

u = x Wup^T, g = x Wgate^T, h = act(g) * u, y = h Wdown^T
(reference: crates/kf-layers/src/ffn.rs:24-47; the activations are those of
crates/kf-backend-cuda/src/kernels/common.cuh:95: gelu_tanh(x) =
0.5 x (1 + tanh(0.79788456 (x + 0.044715 x^3))), gelu_erf, silu).
Gate and up are stacked into one [2*inner, width] matrix when the model is built,
gate rows first, so one product yields both.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, register_feed_forward

ACTIVATIONS = ("gelu_tanh", "gelu_erf", "silu")
GATED_ACTIVATIONS = ACTIVATIONS + ("clamped_swish",)


class GatedFfn(FeedForward):
    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, activation: str = "gelu_tanh", limit: float = 0.0,
                 out_tag: str = "branch_out"):
        """`activation` 'clamped_swish' is the gated form g = min(gate, limit), u = clamp(up, -limit, limit),
        h = g sigmoid(1.702 g) (u + 1) that the experts of some mixtures use (`limit` is read by it alone)."""
        if activation not in GATED_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {GATED_ACTIVATIONS}")
        self.limit, self.out_tag = float(limit), out_tag
        if w_gate_up.dim() == 2 and w_down.dim() == 2 and w_gate_up.shape[0] != 2 * w_down.shape[1]:
            raise ValueError("stacked gate/up matrix must have twice as many rows as the down matrix has columns")
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.activation = activation
        self.inner = w_down.shape[1]
        self.width = w_down.shape[0]

    def forward(self, x, ctx):
        T = x.shape[0]
        h = ctx.buf("ffn_h", (T, self.inner), ctx.act_dtype)
        if self.activation == "clamped_swish":
            ops.linear_gated(x, self.w_gate_up, h, self.activation, ctx, limit=self.limit)
        else:
            ops.linear_gated(x, self.w_gate_up, h, self.activation, ctx)
        y = ctx.buf(self.out_tag, (T, self.width), torch.float32)
        ops.linear(h, self.w_down, y)
        return y


register_feed_forward("gated", GatedFfn)


class DenseFfn(FeedForward):
    """The feed-forward without a gate: y = act(x Wup^T) Wdown^T."""

    def __init__(self, w_up: torch.Tensor, w_down: torch.Tensor, activation: str = "gelu_tanh"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {ACTIVATIONS}")
        if w_up.shape[0] != w_down.shape[1]:
            raise ValueError("the up matrix must have as many rows as the down matrix has columns")
        self.w_up, self.w_down = w_up, w_down
        self.activation = activation
        self.inner = w_down.shape[1]
        self.width = w_down.shape[0]

    def forward(self, x, ctx):
        T = x.shape[0]
        h = ctx.buf("ffn_h", (T, self.inner), ctx.act_dtype)
        ops.linear_act(x, self.w_up, h, self.activation, ctx)
        y = ctx.buf("ffn_out", (T, self.width), torch.float32)
        ops.linear(h, self.w_down, y)
        return y


register_feed_forward("dense", DenseFfn)


class PolyNormFfn(FeedForward):
    """A feed-forward without a gate whose activation norms the powers of its input:
    y = act(x Wup^T) Wdown^T,  act(z) = a N(z) + b N(z^2) + c N(z^3) + e,  N(u) = u / sqrt(mean(u^2) + eps) over a token's
    row, powers element by element, (a, b, c, e) = `coef`.  The up product leaves 32-bit rows; sums and factors are 32-bit."""

    def __init__(self, w_up: torch.Tensor, w_down: torch.Tensor, coef: torch.Tensor, eps: float):
        if w_up.dim() == 2 and w_down.dim() == 2 and w_up.shape[0] != w_down.shape[1]:
            raise ValueError("the up matrix must have as many rows as the down matrix has columns")
        if coef.numel() not in (0, 4):
            raise ValueError(f"the activation takes four numbers, found {coef.numel()}")
        self.w_up, self.w_down, self.coef = w_up, w_down, coef
        self.eps = float(eps)
        self.inner = w_down.shape[1] if w_down.dim() == 2 else 0
        self.width = w_down.shape[0]

    def forward(self, x, ctx):
        T = x.shape[0]
        z = ctx.buf("ffn_up", (T, self.inner), torch.float32)
        ops.linear(x, self.w_up, z)
        h = ctx.buf("ffn_h", (T, self.inner), ctx.act_dtype)
        ops.poly_norm(z, self.coef, self.eps, h)
        y = ctx.buf("ffn_out", (T, self.width), torch.float32)
        ops.linear(h, self.w_down, y)
        return y


register_feed_forward("poly_norm", PolyNormFfn)
