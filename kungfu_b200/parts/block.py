"""How norms, a mixer and a feed-forward stand around the residual stream.

`SandwichBlock` is the arrangement Gemma 2 uses (reference: crates/kf-layers/src/basic.rs:215-265
`Residual` with a post norm, two of them per block, gemma2.rs:39-41):
  h   = x + post_mixer(mixer(pre_mixer(x)))
  out = h + post_ffn(ffn(pre_ffn(h)))
A post norm of None gives the plain pre-norm block other models use; `ffn` None a layer of the first line alone.
The residual stream and its sums stay in 32-bit.
"""
from __future__ import annotations

from .. import ops
from .base import Block, FeedForward, Mixer, Norm, register_block
from .norm import RmsNorm


class SandwichBlock(Block):
    # forward() takes `normed` (this block's pre-mixer norm, already computed by the block before) and `then` (the
    # next block's pre-mixer norm, to be fused into this block's last kernel) and returns (x, normed_for_next)
    fuses_next_norm = True

    def __init__(self, pre_mixer: Norm, mixer: Mixer, post_mixer: Norm | None,
                 pre_ffn: Norm | None, ffn: FeedForward | None, post_ffn: Norm | None):
        self.pre_mixer, self.mixer, self.post_mixer = pre_mixer, mixer, post_mixer
        self.pre_ffn, self.ffn, self.post_ffn = pre_ffn, ffn, post_ffn

    def forward(self, x, ctx, cache, normed=None, then=None):
        act = ctx.act_dtype
        n = normed if normed is not None else self.pre_mixer.forward(x, ctx, act)
        a = self.mixer.forward(n, ctx, cache)
        if self.ffn is None:                                   # a layer without a feed-forward
            if self.post_mixer is not None:
                return x, self.post_mixer.add_into(a, x, ctx, then=then, out_dtype=act if then is not None else None)
            ops.add(a, x)
            return x, (then.forward(x, ctx, act) if then is not None else None)
        if self.post_mixer is not None:
            n = self.post_mixer.add_into(a, x, ctx, then=self.pre_ffn, out_dtype=act)
        else:
            ops.add(a, x)
            n = self.pre_ffn.forward(x, ctx, act)
        f = self.ffn.forward(n, ctx)
        nxt = None
        if self.post_ffn is not None:
            nxt = self.post_ffn.add_into(f, x, ctx, then=then, out_dtype=act if then is not None else None)
        else:
            ops.add(f, x)
            if then is not None:
                nxt = then.forward(x, ctx, act)
        return x, nxt


register_block("sandwich", SandwichBlock)


class ParallelBlock(Block):
    """Mixer and feed-forward side by side on ONE normed input: h = norm(x); x <- x + (mixer(h) + ffn(h)).
    `ffn` may be None (a layer without a feed-forward).  The two branch results and the residual are summed in one
    32-bit kernel that also computes the next block's norm when that is an RMS norm."""
    fuses_next_norm = True

    def __init__(self, norm: Norm, mixer: Mixer, ffn: FeedForward | None):
        self.pre_mixer, self.mixer, self.ffn = norm, mixer, ffn

    def forward(self, x, ctx, cache, normed=None, then=None):
        act = ctx.act_dtype
        h = normed if normed is not None else self.pre_mixer.forward(x, ctx, act)
        a = self.mixer.forward(h, ctx, cache)
        f = self.ffn.forward(h, ctx) if self.ffn is not None else None
        if isinstance(then, RmsNorm):
            nxt = ctx.buf("norm_out", (x.shape[0], then.width), act)       # h is dead once both branches have run
            ops.add2_rmsnorm(a, f, x, next_weight=then.weight, next_eps=then.eps, next_plus_one=then.plus_one, next_out=nxt)
            return x, nxt
        ops.add2_rmsnorm(a, f, x)
        return x, (then.forward(x, ctx, act) if then is not None else None)


register_block("parallel", ParallelBlock)


class ScaledBlock(Block):
    """A pre-norm block whose branch results are multiplied column by column by a learned scale before they join the
    residual, with an optional per-token side input after the feed-forward:
      x <- x + s1 * mixer(norm1(x));   x <- x + s2 * ffn(norm2(x));   x <- x + side_norm(side(x, token))
    `ffn` and `side` may be None.  Every residual update is one 32-bit kernel that also computes the norm that comes next
    (this block's second norm, or the next block's first), and, before a side input, the copy of the residual rows in
    the element type its product takes."""
    fuses_next_norm = True

    def __init__(self, pre_mixer: RmsNorm, mixer: Mixer, scale_mixer, pre_ffn: RmsNorm | None, ffn: FeedForward | None,
                 scale_ffn, side=None):
        self.pre_mixer, self.mixer, self.scale_mixer = pre_mixer, mixer, scale_mixer
        self.pre_ffn, self.ffn, self.scale_ffn, self.side = pre_ffn, ffn, scale_ffn, side

    @staticmethod
    def _norm_args(then, ctx, rows, act):
        if isinstance(then, RmsNorm):
            out = ctx.buf("norm_out", (rows, then.width), act)
            return out, dict(next_weight=then.weight, next_eps=then.eps, next_plus_one=then.plus_one, next_out=out)
        return None, {}

    def forward(self, x, ctx, cache, normed=None, then=None):
        act = ctx.act_dtype
        T = x.shape[0]
        n = normed if normed is not None else self.pre_mixer.forward(x, ctx, act)
        branch, scale = self.mixer.forward(n, ctx, cache), self.scale_mixer
        if self.ffn is not None:
            n2, kw = self._norm_args(self.pre_ffn, ctx, T, act)
            ops.scale_add_rmsnorm(branch, scale, x, **kw)
            branch, scale = self.ffn.forward(n2, ctx), self.scale_ffn
        if self.side is None:
            nxt, kw = self._norm_args(then, ctx, T, act)
            ops.scale_add_rmsnorm(branch, scale, x, **kw)
            if nxt is None and then is not None:
                nxt = then.forward(x, ctx, act)
            return x, nxt
        if act == x.dtype:
            ops.scale_add_rmsnorm(branch, scale, x)
            rows = x
        else:
            rows = ctx.buf("side_rows", tuple(x.shape), act)
            ops.scale_add_rmsnorm(branch, scale, x, copy_out=rows)
        y = self.side.forward(rows, ctx)
        return x, self.side.norm.add_into(y, x, ctx, then=then, out_dtype=act if then is not None else None)


register_block("scaled", ScaledBlock)
