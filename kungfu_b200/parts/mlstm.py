"""A matrix memory with exponential gates (the mLSTM cell of xLSTM) as a mixer.

With H heads, key size d and value size dv, for the input x of a token:
  [q | k | v | g | zi | zf] = x W_in^T          widths H d, H d, H dv, H dv, H, H (one product); q times d^-1/2
  gi = cap tanh((zi + b_i) / cap)                log input gate;  gf = logsigmoid(cap tanh((zf + b_f) / cap))  log forget gate
  m' = max(gf + m, gi)                           running maximum of the gates' logarithms, from 0
  S' = exp(gf + m - m') S + exp(gi - m') k v^T;  n' = exp(gf + m - m') n + exp(gi - m') k          S: d x dv, n: d, from zero
  o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
  o_h <- o_h / sqrt(mean(o_h^2) + eps) * w_h     (one weight vector per head), times sigmoid(g), then y = o W_o^T
The state (S, n, m) is 32-bit and is carried per request in the cache manager's state slots (n in one copy per block of
value columns of the walk: `ops.mlstm_norm_width`), so a request may be fed
in portions of any size; gates, exponentials, the walk, the head norm and the output gate are 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FixedState, Mixer, StateBundle, pad_rows, register_mixer


class MatrixMemory(Mixer):
    def __init__(self, w_in: torch.Tensor, wo: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor,
                 norm_weight: torch.Tensor, *, heads: int, dim: int, vdim: int, gate_cap: float, norm_eps: float,
                 out_tag: str = "branch_out"):
        if dim > 256:
            raise ValueError(f"key size {dim} is above 256, the most the walk keeps in registers")
        if not gate_cap > 0:
            raise ValueError(f"gate_cap must be positive, found {gate_cap}")
        self.wo, self.bias_i, self.bias_f, self.norm_weight = wo, bias_i, bias_f, norm_weight
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        self.gate_cap, self.norm_eps, self.out_tag = float(gate_cap), float(norm_eps), out_tag
        H, d, dv = self.heads, self.dim, self.vdim
        self.q_col, self.k_col, self.v_col = 0, H * d, 2 * H * d
        self.g_col = self.v_col + H * dv
        self.i_col = self.g_col + H * dv
        self.f_col = self.i_col + H
        want = self.f_col + H
        if w_in.numel() and w_in.shape[0] != want:
            raise ValueError(f"the input projection has {w_in.shape[0]} rows, expected {want}")
        self.w_in = pad_rows(w_in)
        self.proj_width = max(want, self.w_in.shape[0])
        self.width = wo.shape[0]

    def state_need(self):
        H, d, dv = self.heads, self.dim, self.vdim
        return StateBundle((FixedState((H, d, dv), torch.float32), FixedState((H, ops.mlstm_norm_width(d, dv)), torch.float32)))

    def forward(self, x, ctx, cache):
        proj = ctx.buf("mlstm_proj", (x.shape[0], self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        return self.forward_projected(proj, 0, ctx, cache)

    @property
    def heads_width(self) -> int:
        """Columns of the output product's input (the normed, gated heads)."""
        return self.heads * self.vdim

    def forward_projected(self, proj, col0: int, ctx, cache, heads_out=None, out_col0: int = 0, scale: float = 1.0):
        """The mixer from its stacked projection's 32-bit result, which starts at column `col0` of `proj`.  With
        `heads_out` it stops before its output product and leaves its normed, gated heads, times `scale`, in columns
        `out_col0`.. of that buffer."""
        memory, norm_state = cache
        T = proj.shape[0]
        H, d, dv = self.heads, self.dim, self.vdim
        o = ctx.buf("mlstm_o", (T, H * dv), torch.float32)
        ops.mlstm(proj, col0 + self.q_col, col0 + self.k_col, col0 + self.v_col, col0 + self.i_col, col0 + self.f_col,
                  self.bias_i, self.bias_f, self.gate_cap, memory.state, norm_state.state, o, H, d, dv, ctx, writes=memory.writes)
        if heads_out is not None:
            ops.head_norm_gate(o, self.norm_weight, self.norm_eps, proj, col0 + self.g_col, "sigmoid", heads_out, H, dv,
                               out_col0=out_col0, scale=scale)
            return None
        normed = ctx.buf("mlstm_normed", (T, H * dv), ctx.act_dtype)
        ops.head_norm_gate(o, self.norm_weight, self.norm_eps, proj, col0 + self.g_col, "sigmoid", normed, H, dv)
        y = ctx.buf(self.out_tag, (T, self.width), torch.float32)
        ops.linear(normed, self.wo, y)
        return y


register_mixer("matrix_memory", MatrixMemory)


class SideBySide(Mixer):
    """Two mixers that read the same input; the result is `left_scale` * left + `right_scale` * right.  Each keeps its
    own state: the cache slot holds both (a bundle, the left mixer's parts first).  Mixers that can start from their
    stacked projection's result (`w_in`, `forward_projected`, `heads_width`, `wo`) share ONE product over both stacked
    input matrices and ONE over both output matrices side by side: each leaves its gated heads, times its scale (in
    32-bit, before the rows are rounded), in its columns of one row, and `[W_o,left | W_o,right]` times that row is the
    weighted sum.  Such mixers belong to this part from then on (their own matrices are released)."""

    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0):
        from ..cache.kinds import flatten_need
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        for m, tag in ((left, "branch_left"), (right, "branch_right")):
            if not hasattr(m, "out_tag"):
                raise ValueError(f"{type(m).__name__} cannot stand beside another mixer: it has no `out_tag`")
            m.out_tag = tag
        self._n_left = len(flatten_need(left.state_need()))
        self._n_right = len(flatten_need(right.state_need()))
        self.w_in = None
        if all(hasattr(m, "forward_projected") and hasattr(m, "w_in") for m in (left, right)):
            a, b = left.w_in, right.w_in
            if a.numel() and b.numel() and a.dtype == b.dtype and a.shape[1] == b.shape[1] and a.shape[0] % 4 == 0:
                self.w_in = torch.cat([a, b], dim=0).contiguous()       # the right mixer's columns start on a 16-byte boundary
                self._right_col0 = a.shape[0]
                left.w_in, right.w_in = self.w_in[: a.shape[0]], self.w_in[a.shape[0]:]     # views: the weights are held once
        self.wo = None
        if self.w_in is not None and all(hasattr(m, "heads_width") and hasattr(m, "wo") for m in (left, right)):
            a, b = left.wo, right.wo
            if a.numel() and b.numel() and a.dtype == b.dtype and a.shape[0] == b.shape[0]:
                self.wo = torch.cat([a, b], dim=1).contiguous()         # [width, left heads | right heads]
                self._k_left = a.shape[1]
                left.wo = right.wo = a.new_empty(0)                     # held once, side by side

    def state_need(self):
        parts = tuple(n for n in (self.left.state_need(), self.right.state_need()) if n is not None)
        if not parts:
            return None
        return parts[0] if len(parts) == 1 else StateBundle(parts)

    @staticmethod
    def _views(views: tuple, need):
        if need is None:
            return None
        return views if isinstance(need, StateBundle) else views[0]

    def forward(self, x, ctx, cache):
        views = cache if isinstance(cache, tuple) else ((cache,) if cache is not None else ())
        lv = self._views(views[: self._n_left], self.left.state_need())
        rv = self._views(views[self._n_left:], self.right.state_need())
        if self.w_in is not None:
            proj = ctx.buf("side_proj", (x.shape[0], self.w_in.shape[0]), torch.float32)
            ops.linear(x, self.w_in, proj)
            if self.wo is not None:
                heads = ctx.buf("side_heads", (x.shape[0], self.wo.shape[1]), ctx.act_dtype)
                self.left.forward_projected(proj, 0, ctx, lv, heads_out=heads, out_col0=0, scale=self.left_scale)
                self.right.forward_projected(proj, self._right_col0, ctx, rv, heads_out=heads, out_col0=self._k_left,
                                             scale=self.right_scale)
                y = ctx.buf("branch_out", (x.shape[0], self.wo.shape[0]), torch.float32)
                ops.linear(heads, self.wo, y)
                return y
            a = self.left.forward_projected(proj, 0, ctx, lv)
            b = self.right.forward_projected(proj, self._right_col0, ctx, rv)
        else:
            a = self.left.forward(x, ctx, lv)
            b = self.right.forward(x, ctx, rv)
        y = ctx.buf("branch_out", tuple(a.shape), torch.float32)
        ops.weighted_sum2(a, self.left_scale, b, self.right_scale, y)
        return y


register_mixer("side_by_side", SideBySide)
