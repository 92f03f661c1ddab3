"""Root-mean-square norm.

y_i = x_i / sqrt(mean_j(x_j^2) + eps) * g_i with g = w, or g = 1 + w when `plus_one`
(reference: crates/kf-backend-cuda/src/kernels/norm.cu:4-14 for the norm and :16-27 for
the norm that is added to the residual; Gemma 2 files store w and use 1 + w).
Sums, the reciprocal root and the product run in 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, register_norm


class RmsNorm(Norm):
    def __init__(self, weight: torch.Tensor, eps: float, plus_one: bool = False):
        self.weight = weight
        self.eps = float(eps)
        self.plus_one = bool(plus_one)
        self.width = weight.shape[0]

    def forward(self, x, ctx, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buf("norm_out" if rows is None else "norm_rows_out", (n, self.width), out_dtype)
        ops.rmsnorm(x, self.weight, self.eps, self.plus_one, out, rows)
        return out

    def add_into(self, branch, residual, ctx, then=None, out_dtype=None):
        """residual += norm(branch); returns then(residual) if `then` is given (one kernel when `then` is an RmsNorm)."""
        if then is None:
            ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual)
            return None
        if isinstance(then, RmsNorm):
            out = ctx.buf("norm_out", (residual.shape[0], self.width), out_dtype)
            ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual,
                            next_weight=then.weight, next_eps=then.eps, next_plus_one=then.plus_one, next_out=out)
            return out
        if isinstance(then, NoNorm) and out_dtype != residual.dtype:
            out = ctx.buf("norm_out", (residual.shape[0], self.width), out_dtype)       # the sum and the copy in one kernel
            ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual, copy_out=out)
            return out
        ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual)
        return then.forward(residual, ctx, out_dtype)


register_norm("rms", RmsNorm)


class GroupRmsNorm(Norm):
    """RMS norm in groups: the row is cut into `groups` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps); the whole row is then multiplied by the weight.  One group is the plain RMS norm."""

    def __init__(self, weight: torch.Tensor, eps: float, groups: int = 1):
        self.weight = weight
        self.eps = float(eps)
        self.groups = int(groups)
        self.width = weight.shape[0]
        if self.groups < 1 or (self.width and self.width % self.groups):
            raise ValueError(f"a row of {self.width} cannot be cut into {self.groups} equal parts")

    def forward(self, x, ctx, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buf("norm_out" if rows is None else "norm_rows_out", (n, self.width), out_dtype)
        ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out, rows)
        return out

    def _fuses(self, then) -> bool:
        return isinstance(then, GroupRmsNorm) and then.groups == self.groups and then.weight.dtype == self.weight.dtype

    def add_into(self, branch, residual, ctx, then=None, out_dtype=None):
        """residual += norm(branch); returns then(residual) if `then` is given (one kernel when `then` cuts rows alike)."""
        if then is not None and self._fuses(then):
            out = ctx.buf("norm_out", (residual.shape[0], self.width), out_dtype)
            ops.add_group_rmsnorm(branch, self.weight, self.eps, self.groups, residual, next_weight=then.weight,
                                  next_eps=then.eps, next_out=out)
            return out
        ops.add_group_rmsnorm(branch, self.weight, self.eps, self.groups, residual)
        return then.forward(residual, ctx, out_dtype) if then is not None else None

    def after_shift(self, residual, shift, ctx, out_dtype):
        """residual += shift (one constant row for all rows); returns norm(residual).  One kernel."""
        out = ctx.buf("norm_out", (residual.shape[0], self.width), out_dtype)
        ops.add_group_rmsnorm(None, None, 0.0, self.groups, residual, shift=shift, next_weight=self.weight, next_eps=self.eps,
                              next_out=out)
        return out


register_norm("group_rms", GroupRmsNorm)


class NoNorm(Norm):
    """The place of a norm in a block whose sublayers read the residual stream itself: the rows pass unchanged, in the
    element type the sublayer's products take (the residual's own rows when that is 32-bit)."""

    def __init__(self, width: int):
        self.width = int(width)

    def forward(self, x, ctx, out_dtype, rows=None):
        if rows is not None:
            raise NotImplementedError("NoNorm passes whole steps only")
        if out_dtype == x.dtype:
            return x
        out = ctx.buf("norm_out", (x.shape[0], self.width), out_dtype)
        ops.convert(x, out)
        return out


register_norm("none", NoNorm)
