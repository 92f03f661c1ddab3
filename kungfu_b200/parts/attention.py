"""Grouped-query attention over paged keys and values.

In order (reference: crates/kf-layers/src/attention.rs:118-150,160-172,211-283 and
crates/kf-backend-cpu/src/attention.rs:33-45,79-147):
  q, k, v = x Wq^T, x Wk^T, x Wv^T (one product over the stacked matrix)
  q, k rotated by the position encoding; k, v written to the request's pages at the token's position
  head h reads kv head h / (n_heads / n_kv_heads)
  s_j = (q . k_j) * scale; if softcap: s_j = cap * tanh(s_j / cap)
  key j is seen from position p iff j <= p and (no window or p - j < window)
  o = sum_j softmax(s)_j v_j (zeros when no key is seen); y = o Wo^T
Scores, the softmax and the weighted sum are 32-bit.  Sizes and constants are arguments:
this part does not know which model it sits in.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedKV, PositionEncoding, StateBundle, pad_rows, register_mixer
from .conv import ShortConv


class PagedAttention(Mixer):
    def __init__(self, wqkv: torch.Tensor, wo: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, softcap: float = 0.0, window: int | None = None,
                 position: PositionEncoding | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        self.wqkv, self.wo = wqkv, wo
        self.n_heads, self.n_kv_heads, self.head_dim = int(n_heads), int(n_kv_heads), int(head_dim)
        self.scale, self.softcap = float(scale), float(softcap)
        self.window = None if window is None else int(window)
        self.position = position
        self.width = wo.shape[0]
        ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim)

    def state_need(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        nh, nkv, d = self.n_heads, self.n_kv_heads, self.head_dim
        if self.position is not None:
            cos, sin = self.position.rotation(ctx)
            rot = 2 * cos.shape[1]
        else:
            cos = sin = None
            rot = 0
        o = ctx.buf("attn_o", (T, nh * d), ctx.act_dtype)
        if ops.decode_attention_takes_qkv(ctx, cache, nh, nkv, d):
            # a decode step: the attention kernel rotates, appends and attends in one launch
            qkv = ctx.buf("attn_qkv", (T, (nh + 2 * nkv) * d), torch.float32)
            ops.linear(x, self.wqkv, qkv)
            ops.rope_append_attend(qkv, cos, sin, rot, o, ctx, cache, nh, nkv, d, self.scale, self.softcap, self.window)
        else:
            q = ctx.buf("attn_q", (T, nh * d), ctx.act_dtype)
            # a long prompt: the product rotates and files its own result where it can
            if not ops.linear_rope_kv_append(x, self.wqkv, cos, sin, rot, nh, nkv, d, ctx, cache, q):
                qkv = ctx.buf("attn_qkv", (T, (nh + 2 * nkv) * d), torch.float32)
                ops.linear(x, self.wqkv, qkv)
                ops.rope_kv_append(qkv, cos, sin, rot, nh, nkv, d, ctx, cache, q)
            ops.paged_attention(q, o, ctx, cache, nh, nkv, d, self.scale, self.softcap, self.window)
        y = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(o, self.wo, y)
        return y


register_mixer("paged_attention", PagedAttention)


class ConvGatedAttention(Mixer):
    """Grouped-query attention whose q, k and v pass more than a rotation on their way from the projection, and whose
    heads are gated on their way out.  In order, every step optional except the attention itself:

      [q | k | v | g] = x W_in^T (+ bias on q, k, v)          one product over the stacked matrix
      q, k, v <- short causal convolution over time, per channel (`conv`, state: the last taps - 1 projected rows)
      q, k <- RMS norm over each head, one weight vector for all heads (`q_norm`, `k_norm`)
      q, k <- rotation of the first rotary dims by `position` (its `interleaved` flag chooses the pairing)
      k, v written to the request's pages; o = softmax(softcap(q . k * scale)) v, causal, optionally windowed
      o_h <- o_h * sigmoid(g_h)                                one gate per head, from the same input x
      y = o W_o^T

    Keys and values may have different head sizes (`key_dim`, `value_dim`); the cache holds heads of
    D = max of the two (rounded up to even) with zero tails, so the framework's attention kernels serve both.
    Scores, softmax, norms, the rotation and the gate are 32-bit."""

    def __init__(self, w_in: torch.Tensor, wo: torch.Tensor, *, n_heads: int, n_kv_heads: int, key_dim: int,
                 value_dim: int, scale: float, softcap: float = 0.0, window: int | None = None,
                 position: PositionEncoding | None = None, bias: torch.Tensor | None = None,
                 conv: ShortConv | None = None, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                 norm_eps: float = 1e-6, gated: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        self.w_in, self.wo, self.bias = w_in, wo, bias
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)
        self.key_dim, self.value_dim = int(key_dim), int(value_dim)
        self.head_dim = (max(self.key_dim, self.value_dim) + 1) // 2 * 2
        self.scale, self.softcap = float(scale), float(softcap)
        self.window = None if window is None else int(window)
        self.position, self.conv = position, conv
        self.q_norm, self.k_norm, self.norm_eps = q_norm, k_norm, float(norm_eps)
        self.gated = bool(gated)
        self.qkv_width = (self.n_heads + self.n_kv_heads) * self.key_dim + self.n_kv_heads * self.value_dim
        self.proj_width = self.qkv_width + (self.n_heads if self.gated else 0)
        self.width = wo.shape[0]
        if w_in.numel() and w_in.shape[0] != self.proj_width:
            raise ValueError(f"stacked projection has shape {tuple(w_in.shape)}, expected {self.proj_width} rows")
        self.w_in = pad_rows(w_in)                          # result rows start on 16-byte boundaries
        self.proj_width = max(self.proj_width, self.w_in.shape[0])
        if conv is not None and conv.channels != self.qkv_width:
            raise ValueError(f"the convolution has {conv.channels} channels, q|k|v have {self.qkv_width}")
        rot = getattr(position, "rotary_dims", 0) if position is not None else 0
        if rot > self.key_dim:
            raise ValueError(f"{rot} rotary dims for keys of {self.key_dim}")
        ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim)

    def state_need(self):
        kv = PagedKV(self.n_kv_heads, self.head_dim, self.window)
        if self.conv is None or self.conv.taps <= 1:
            return kv
        return StateBundle((kv, self.conv.state_need()))

    def forward(self, x, ctx, cache):
        kv, tail = cache if isinstance(cache, tuple) else (cache, None)
        T = x.shape[0]
        nh, nkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        proj = ctx.buf("attn_proj", (T, self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        if self.position is not None:
            cos, sin = self.position.rotation(ctx)
            rot, interleaved = 2 * cos.shape[1], bool(getattr(self.position, "interleaved", False))
        else:
            cos = sin = None
            rot, interleaved = 0, False
        q = ctx.buf("attn_q", (T, nh * D), ctx.act_dtype)
        conv = self.conv
        moves = tail is not None and tail.writes
        done = ops.qkv_prepare(proj, 0, self.bias, conv.weight if conv else None, tail.state if tail is not None else None,
                               self.q_norm, self.k_norm, self.norm_eps, cos, sin, rot, interleaved, nh, nkv, self.key_dim,
                               self.value_dim, ctx, kv, q, commit_inline=moves and bool(getattr(ctx, "decode_only", False)))
        if moves and not done:
            conv.commit(proj, 0, self.bias, ctx, tail)
        o = ctx.buf("attn_o", (T, nh * D), ctx.act_dtype)
        ops.paged_attention(q, o, ctx, kv, nh, nkv, D, self.scale, self.softcap, self.window)
        if self.gated or D != self.value_dim:
            packed = ctx.buf("attn_gated", (T, nh * self.value_dim), ctx.act_dtype)
            ops.head_gate(o, proj if self.gated else None, self.qkv_width, nh, self.value_dim, D, packed, ctx)
            o = packed
        y = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(o, self.wo, y)
        return y


register_mixer("conv_gated_attention", ConvGatedAttention)


class TalkingAttention(Mixer):
    """Grouped-query attention with unit-norm queries and keys, whose softmax weights are mixed across heads after the
    softmax, and whose heads are gated element by element on their way out.  In order, for the normed input x:

      [q | k | v | g] = x W_in^T                                one product over the stacked matrix
      q, k <- rotation of the first rotary dims by `position`, pairs (i, i + rot/2), cos and sin times its `magnitude`
      q, k <- head / sqrt(mean(head^2) + norm_eps)              after the rotation, no weight (`unit_norm`)
      a_h(i, .) = softmax_j(q_h(i) . k_(h/r)(j) * scale), causal, optionally windowed;  r = n_heads / n_kv_heads
      b_h = sum_g mix[h, g] a_g                                 the heads' weights mixed (`mix` [n_heads, n_heads])
      o_h(i) = sum_j b_h(i, j) v_(h/r)(j)
      o <- o * sigmoid(g)                                       one gate per element, from the same input x
      y = o W_o^T

    Since o_h = sum_g mix[h, g] O[g, h/r] with O[g, c] the plain attention of query head g over value head c, the
    framework's attention kernels do the work: they give every query head's weighted sum over every value head
    (`ops.paged_attention(value_split=n_kv_heads)`, n_heads * n_kv_heads result heads from the same queries and pages);
    `ops.head_mix_gate` then sums over g and gates.  The cache holds n_kv_heads heads of D = max(key_dim, value_dim),
    rounded up to a size the kernels take.  With `mix` None the mixer is plain grouped-query attention with
    the same extras.  Scores, softmax, norms, rotation, mixing sums and the gate are 32-bit."""

    def __init__(self, w_in: torch.Tensor, wo: torch.Tensor, *, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, window: int | None = None, position: PositionEncoding | None = None,
                 mix: torch.Tensor | None = None, unit_norm: bool = True, norm_eps: float = 1e-6, gated: bool = True):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        self.wo, self.mix = wo, mix
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)
        self.key_dim, self.value_dim = int(key_dim), int(value_dim)
        self.head_dim = ops.attention_head_size(max(self.key_dim, self.value_dim))
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.position = position
        self.unit_norm, self.norm_eps, self.gated = bool(unit_norm), float(norm_eps), bool(gated)
        self.reps = self.n_kv_heads if mix is not None else 1
        self.qkv_width = (self.n_heads + self.n_kv_heads) * self.key_dim + self.n_kv_heads * self.value_dim
        self.proj_width = self.qkv_width + (self.n_heads * self.value_dim if self.gated else 0)
        self.width = wo.shape[0]
        if w_in.numel() and w_in.shape[0] != self.proj_width:
            raise ValueError(f"stacked projection has shape {tuple(w_in.shape)}, expected {self.proj_width} rows")
        if mix is not None and mix.numel() and tuple(mix.shape) != (self.n_heads, self.n_heads):
            raise ValueError(f"the mixing matrix has shape {tuple(mix.shape)}, expected {(self.n_heads, self.n_heads)}")
        self.w_in = pad_rows(w_in)
        self.proj_width = max(self.proj_width, self.w_in.shape[0])
        rot = getattr(position, "rotary_dims", 0) if position is not None else 0
        if rot > self.key_dim:
            raise ValueError(f"{rot} rotary dims for keys of {self.key_dim}")
        if position is not None and getattr(position, "interleaved", False):
            raise ValueError("this mixer turns pairs (i, i + rot/2); an interleaved rotation is not supported")
        ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim)

    def state_need(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        nh, nkv, D, reps = self.n_heads, self.n_kv_heads, self.head_dim, self.reps
        proj = ctx.buf("attn_proj", (T, self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        if self.position is not None:
            cos, sin = self.position.rotation(ctx)
            rot, mag = 2 * cos.shape[1], float(getattr(self.position, "magnitude", 1.0))
        else:
            cos = sin = None
            rot, mag = 0, 1.0
        q = ctx.buf("attn_q", (T, nh * D), ctx.act_dtype)
        ops.rotate_norm_append(proj, 0, cos, sin, rot, mag, self.unit_norm, self.norm_eps, nh, nkv, self.key_dim,
                               self.value_dim, ctx, cache, q)
        o = ctx.buf("attn_o", (T, nh * reps * D), ctx.act_dtype)
        if self.mix is not None:
            ops.paged_attention(q, o, ctx, cache, nh * nkv, nkv * nkv, D, self.scale, 0.0, self.window, value_split=nkv)
        else:
            ops.paged_attention(q, o, ctx, cache, nh, nkv, D, self.scale, 0.0, self.window)
        if self.mix is not None or self.gated or D != self.value_dim:
            packed = ctx.buf("attn_gated", (T, nh * self.value_dim), ctx.act_dtype)
            ops.head_mix_gate(o, self.mix, proj if self.gated else None, self.qkv_width, nh, nkv, self.value_dim, D, packed, ctx)
            o = packed
        y = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(o, self.wo, y)
        return y


register_mixer("talking_attention", TalkingAttention)


class RowNormAttention(Mixer):
    """Grouped-query attention whose q and k are normed over the WHOLE projection (all heads of a row at once), with
    optional extras.  In order, for the input x:

      [q | k | v | g] = x W_in^T (+ bias on q, k, v)            one product over the stacked matrix
      q <- q / sqrt(mean over all of q's elements of q^2 + eps) * q_norm;  k likewise        (`q_norm`, `k_norm`: weights of
                                                                 n_heads * key_dim and n_kv_heads * key_dim; None: no norm)
      q, k <- rotation of the first rotary dims of every head by `position` (its `interleaved` flag chooses the pairing)
      v <- (1 - lambda) v + lambda v_first                      `v_mix` "mix": v_first = the biased v of the same token in
                                                                 the layer whose `v_mix` is "first" and whose `v_mix_tag`
                                                                 is the same; the mixed v is what the pages hold
      s_j = (q . k_j) * scale; key j is seen from position p iff j <= p and (no window, or p - j < window, or j < keep_first)
      a = exp(s_j) / (sum exp(s) + 1 if `sink` else sum exp(s))
      o_h <- o_h * sigmoid(g_h)                                  one gate per head, from the same input x (`gated`)
      y = o W_o^T
    Scores, softmax, norms, rotation, mixing and gate are 32-bit."""

    def __init__(self, w_in: torch.Tensor, wo: torch.Tensor, *, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, window: int | None = None, keep_first: int = 0, sink: bool = False,
                 position: PositionEncoding | None = None, bias: torch.Tensor | None = None,
                 q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None, norm_eps: float = 1e-6,
                 gated: bool = False, v_mix: str | None = None, v_mix_weight: torch.Tensor | None = None,
                 v_mix_tag: str = "v_first", out_tag: str = "branch_out"):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        if v_mix not in (None, "first", "mix"):
            raise ValueError(f"v_mix {v_mix!r} is not one of None, 'first', 'mix'")
        self.wo, self.bias = wo, bias
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)
        self.key_dim, self.value_dim = int(key_dim), int(value_dim)
        self.head_dim = ops.attention_head_size(max(self.key_dim, self.value_dim))
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.keep_first = int(keep_first) if self.window is not None else 0
        self.sink = bool(sink)
        self.position = position
        self.q_norm, self.k_norm, self.norm_eps = q_norm, k_norm, float(norm_eps)
        self.gated = bool(gated)
        self.v_mix, self.v_mix_tag, self.out_tag = v_mix, v_mix_tag, out_tag
        self.v_mix_weight = v_mix_weight.reshape(-1).contiguous() if (v_mix_weight is not None and v_mix_weight.numel()) else None
        if v_mix == "mix" and self.v_mix_weight is None and (v_mix_weight is None):
            raise ValueError("v_mix 'mix' needs the mixing number")
        self.qkv_width = (self.n_heads + self.n_kv_heads) * self.key_dim + self.n_kv_heads * self.value_dim
        self.proj_width = self.qkv_width + (self.n_heads if self.gated else 0)
        self.width = wo.shape[0]
        if w_in.numel() and w_in.shape[0] != self.proj_width:
            raise ValueError(f"stacked projection has shape {tuple(w_in.shape)}, expected {self.proj_width} rows")
        self.w_in = pad_rows(w_in)
        self.proj_width = max(self.proj_width, self.w_in.shape[0])
        rot = getattr(position, "rotary_dims", 0) if position is not None else 0
        if rot > self.key_dim:
            raise ValueError(f"{rot} rotary dims for keys of {self.key_dim}")
        ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim)

    def state_need(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window, self.keep_first)

    def forward(self, x, ctx, cache):
        proj = ctx.buf("attn_proj", (x.shape[0], self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        return self.forward_projected(proj, 0, ctx, cache)

    @property
    def heads_width(self) -> int:
        """Columns of the output product's input (the gated heads)."""
        return self.n_heads * self.value_dim

    def forward_projected(self, proj, col0: int, ctx, cache, heads_out=None, out_col0: int = 0, scale: float = 1.0):
        """The mixer from its stacked projection's 32-bit result, which starts at column `col0` of `proj` (a mixer that
        stands beside another one shares one product over both stacked matrices).  With `heads_out` the mixer stops before
        its output product and leaves its gated heads, times `scale`, in columns `out_col0`.. of that buffer (the other
        mixer's follow, and one product over both output matrices side by side gives the weighted sum)."""
        T = proj.shape[0]
        nh, nkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        if self.position is not None:
            cos, sin = self.position.rotation(ctx)
            rot, interleaved = 2 * cos.shape[1], bool(getattr(self.position, "interleaved", False))
            mag = float(getattr(self.position, "magnitude", 1.0))
        else:
            cos = sin = None
            rot, interleaved, mag = 0, False, 1.0
        q = ctx.buf("attn_q", (T, nh * D), ctx.act_dtype)
        shared, mode = None, 0
        if self.v_mix is not None:
            shared = ctx.buf(f"attn_{self.v_mix_tag}", (T, nkv * self.value_dim), torch.float32)
            mode = 1 if self.v_mix == "first" else 2
        ops.rownorm_rope_append(proj, col0, self.bias, self.q_norm, self.k_norm, self.norm_eps, cos, sin, rot, interleaved, mag,
                                nh, nkv, self.key_dim, self.value_dim, ctx, cache, q,
                                v_mix=self.v_mix_weight if mode == 2 else None, v_shared=shared, v_mode=mode)
        o = ctx.buf("attn_o", (T, nh * D), ctx.act_dtype)
        ops.paged_attention(q, o, ctx, cache, nh, nkv, D, self.scale, 0.0, self.window, keep_first=self.keep_first,
                            sink=self.sink)
        if heads_out is not None:                      # the gated heads, times `scale`, into a row another product reads
            ops.head_gate(o, proj if self.gated else None, col0 + self.qkv_width, nh, self.value_dim, D, heads_out, ctx,
                          out_col0=out_col0, scale=scale)
            return None
        if self.gated or D != self.value_dim:
            packed = ctx.buf("attn_gated", (T, nh * self.value_dim), ctx.act_dtype)
            ops.head_gate(o, proj if self.gated else None, col0 + self.qkv_width, nh, self.value_dim, D, packed, ctx)
            o = packed
        y = ctx.buf(self.out_tag, (T, self.width), torch.float32)
        ops.linear(o, self.wo, y)
        return y


register_mixer("row_norm_attention", RowNormAttention)
