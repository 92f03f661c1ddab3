"""A mixture of experts: a router picks a few small gated feed-forwards per token; a shared one may run for all.

For the normed input x of a token, with E experts of which `top` are used:
  z = W_r x (32-bit);  s = sigmoid(z);  choice = s + correction        (the correction steers the choice only)
  experts stand in `groups` equal groups of neighbours; a group's score is the sum of its two largest choice scores;
  only experts of the `keep` best groups are eligible; the `top` largest eligible choice scores win
  weight_e = s_e / (sum of the winners' s + 1e-20) * scale
  expert_e(x) = W_down,e [ g sigmoid(1.702 g) (u + 1) ],  g = min(W_gate,e x, limit),  u = clamp(W_up,e x, -limit, limit)
  y = sum over winners of weight_e expert_e(x)  (+ shared(x), an expert of the same form with sizes and limit of its own)
On the device the (token, choice) pairs are laid out expert by expert (`ops.moe_plan`), the experts' two products run as
grouped products over that layout, and the weighted sum walks each token's choices in order: a token's result does not
depend on what else is in the step.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, register_feed_forward


class RoutedExperts(FeedForward):
    def __init__(self, w_router: torch.Tensor, correction: torch.Tensor | None, w_gate_up: torch.Tensor, w_down: torch.Tensor, *,
                 top: int, scale: float, limit: float, groups: int = 1, keep: int = 1, shared: FeedForward | None = None,
                 score: str = "sigmoid", group_rank: str = "best_two", normalize: bool = True,
                 activation: str = "clamped_swish", weight_on: str = "output"):
        """w_gate_up [E, 2 ff, width] (gate rows, then up rows, per expert), w_down [E, width, ff].
        Other mixtures of the same shape: `score` 'softmax' (scores = the softmax of z over all experts), `group_rank`
        'best' (a group scores its largest member), `normalize` False (the winners keep their scores as weights, times
        `scale`), `activation` 'silu' (experts W_down [silu(g) u]), `weight_on` 'input' (y = sum of expert_e(weight_e x):
        the weight multiplies what the expert reads, i.e. its gate and up rows before the activation, not its result)."""
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on {weight_on!r} is not one of output, input")
        self.weight_on = weight_on
        if score not in ("sigmoid", "softmax") or group_rank not in ("best_two", "best") or activation not in ("clamped_swish", "silu"):
            raise ValueError(f"score {score!r}, group_rank {group_rank!r} or activation {activation!r} is not known")
        self.score, self.group_rank, self.normalize, self.activation = score, group_rank, bool(normalize), activation
        self.w_router, self.correction = w_router, correction
        self.w_gate_up, self.w_down, self.shared = w_gate_up, w_down, shared
        self.top, self.scale, self.limit = int(top), float(scale), float(limit)
        self.groups, self.keep = int(groups), int(keep)
        self.n_experts = int(w_router.shape[0]) if w_router.numel() else 0
        E = self.n_experts
        if E:
            if not (1 <= self.top <= E):
                raise ValueError(f"top {self.top} of {E} experts")
            if self.groups < 1 or E % self.groups or not (1 <= self.keep <= self.groups):
                raise ValueError(f"{E} experts do not form {self.groups} equal groups of which {self.keep} stay")
            if self.groups > 1 and self.keep * (E // self.groups) < self.top:
                raise ValueError(f"{self.keep} groups of {E // self.groups} experts cannot give {self.top} choices")
        self.inner = int(w_down.shape[2]) if w_down.dim() == 3 else 0
        self.width = int(w_down.shape[1]) if w_down.dim() == 3 else 0

    def forward(self, x, ctx):
        T = x.shape[0]
        E, top = self.n_experts, self.top
        logits = ctx.buf("moe_logits", (T, E), torch.float32)
        ops.linear(x, self.w_router, logits)
        ids = ctx.buf("moe_ids", (T, top), torch.int32)
        wts = ctx.buf("moe_weights", (T, top), torch.float32)
        ops.moe_route(logits, self.correction, self.groups, self.keep, top, self.scale, ids, wts, score=self.score,
                      group_rank=self.group_rank, normalize=self.normalize)
        plan = ops.moe_plan(ids, E, ctx)
        h = ctx.buf("moe_h", (T * top, self.inner), ctx.act_dtype)
        on_input = self.weight_on == "input"
        ops.moe_linear(x, plan, self.w_gate_up, h, gather=True, gated=True, limit=self.limit, activation=self.activation,
                       row_scale=wts if on_input else None)
        eo = ctx.buf("moe_expert_out", (T * top, self.width), torch.float32)
        ops.moe_linear(h, plan, self.w_down, eo, gather=False)
        sh = self.shared.forward(x, ctx) if self.shared is not None else None
        y = ctx.buf("ffn_out", (T, self.width), torch.float32)
        ops.moe_combine(eo, plan, None if on_input else wts, sh, y)
        return y


register_feed_forward("routed_experts", RoutedExperts)
