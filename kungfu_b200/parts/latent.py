"""Attention over a latent: every token leaves one small row c in the cache, and every head's keys and values are linear
maps of it.

For the normed input x of a token, with H heads, query/key size d, value size dv and latent size r:
  q_h = W_q,h x                                  c = rms_norm(W_dkv x) * w_c            (only c is cached, in pages)
  k_h(j) = W_uk,h c_j,  v_h(j) = W_uv,h c_j      s_hj = (q_h . k_h(j)) * scale, causal softmax over j, no positions
  y = W_o concat_h(sum_j p_hj v_h(j))
The expansions never happen.  Because q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j and sum_j p_hj W_uv,h c_j =
W_uv,h (sum_j p_hj c_j), the mixer maps each query into the latent space (one small product per head), runs the
framework's paged attention with ONE key/value head whose key row and value row are both c_j, and maps each head's
result back with W_uv,h.  The latent head is padded with zeros to the next size the attention kernels have an instance
for (the maps' weights are padded likewise, so the padding is exact).  Scores, softmax and the norm of c are 32-bit.

Options for other models of the kind:
  `w_dq`, `dq_norm`   queries through a latent of their own: c_q = rms_norm(W_dq x) * w_q, q = W_q c_q (W_q then maps the
                      query latent to the heads)
  `rot_dim`, `position`  every head's query has `rot_dim` more elements behind its `dim`, and W_dkv x has `rot_dim` more
                      rows behind the latent: one key part shared by all heads.  Both are turned by `position` and their
                      dot product is added to the score: s = (q_h . W_uk,h c + q_rot,h . k_rot) * scale.  In the latent
                      space the shared part simply rides behind c in the stored key row (zeros in the value row) and
                      behind W_uk,h^T q_h in the query.
  `w_gate`            head h's result is multiplied by sigmoid(W_g x)_h before the output projection.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedKV, PositionEncoding, pad_rows, register_mixer

_KERNEL_HEAD_SIZES = (16, 32, 64, 128, 256, 384, 512)          # above 256 the generic attention kernel alone


def latent_head_size(rank: int) -> int:
    """The head size the latent is stored with: the smallest the tensor-core attention kernels take that holds `rank`."""
    for d in _KERNEL_HEAD_SIZES:
        if rank <= d:
            return d
    raise ValueError(f"a latent of {rank} elements is above {_KERNEL_HEAD_SIZES[-1]}, the largest head the attention kernels take")


class _RowsAsParts:
    """A decode step seen by the attention kernels as `parts` rows per token, each with 1 / parts of the heads: the same
    pages and block tables, positions and requests repeated.  (The tensor-core decode kernel takes the query heads of
    one key/value head as the rows of ONE 16-row tile; a latent has a single key/value head for all heads.)"""

    def __init__(self, ctx, parts: int):
        T = ctx.n_rows
        self.positions = ctx.buf("latent_positions", (T * parts,), torch.int32)
        self.row_req = ctx.buf("latent_row_req", (T * parts,), torch.int32)
        ops.repeat_rows(ctx.positions, ctx.row_req, parts, self.positions, self.row_req)
        self.block_tables, self.max_kv_len = ctx.block_tables, ctx.max_kv_len
        self.n_rows = self.n_dec_rows = T * parts
        self.n_pre_rows = self.n_tiles = self.n_wide = 0
        self.dec_rows = self.pre_rows = None


def _decode_parts(n_heads: int) -> int:
    """Into how many parts the heads are cut for decode steps: the fewest that leave at most 16 heads each."""
    for parts in range(1, n_heads + 1):
        if n_heads % parts == 0 and n_heads // parts <= 16:
            return parts
    return 1


class LatentAttention(Mixer):
    def __init__(self, w_q: torch.Tensor, w_dkv: torch.Tensor, c_norm: torch.Tensor, w_uk: torch.Tensor, w_uv: torch.Tensor,
                 wo: torch.Tensor, *, n_heads: int, dim: int, vdim: int, rank: int, scale: float, norm_eps: float,
                 window: int | None = None, w_dq: torch.Tensor | None = None, dq_norm: torch.Tensor | None = None,
                 rot_dim: int = 0, position: PositionEncoding | None = None, w_gate: torch.Tensor | None = None,
                 out_tag: str = "branch_out"):
        self.n_heads, self.dim, self.vdim, self.rank = int(n_heads), int(dim), int(vdim), int(rank)
        self.rot_dim = int(rot_dim) if position is not None else 0
        self.position = position
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.window = None if window is None else int(window)
        self.head_dim = D = latent_head_size(self.rank + self.rot_dim)
        self.width = wo.shape[0]
        self.c_norm, self.wo, self.dq_norm, self.out_tag = c_norm, wo, dq_norm, out_tag
        self.q_latent = w_dq is not None
        self.gated = w_gate is not None
        H, d, dv, r, rd = self.n_heads, self.dim, self.vdim, self.rank, self.rot_dim
        self.q_rank = int(w_dq.shape[0]) if (self.q_latent and w_dq.numel()) else 0
        given = [w_q, w_dkv, w_uk, w_uv] + ([w_dq] if self.q_latent else []) + ([w_gate] if self.gated else [])
        if all(t.numel() for t in given):
            # one product of the input: [q or the query latent | c and the shared key part | gate]
            first = [w_dq if self.q_latent else w_q, w_dkv] + ([w_gate] if self.gated else [])
            self.w_in = pad_rows(torch.cat(first, dim=0).contiguous())
            self.w_uq = w_q if self.q_latent else None
            # W_uk,h^T as a map (d + rd) -> D: the unrotated part into the latent's places, the rotated part, unchanged,
            # into the places behind them (rows beyond r + rd zero); W_uv,h as a map D -> dv (columns beyond r zero)
            uk = torch.zeros((H, D, d + rd), dtype=w_uk.dtype, device=w_uk.device)
            uk[:, :r, :d] = w_uk.view(H, d, r).transpose(1, 2)
            for i in range(rd):
                uk[:, r + i, d + i] = 1.0
            uv = torch.zeros((H, dv, D), dtype=w_uv.dtype, device=w_uv.device)
            uv[:, :, :r] = w_uv.view(H, dv, r)
            self.w_uk_t, self.w_uv = uk.contiguous(), uv.contiguous()
        else:                                              # a fault the weight store has already recorded
            self.w_in = self.w_uk_t = self.w_uv = torch.empty(0)
            self.w_uq = None
        self.q_width = H * (d + rd)
        self.c_col = self.q_rank if self.q_latent else self.q_width
        self.g_col = self.c_col + r + rd
        self.proj_width = max(self.g_col + (H if self.gated else 0), self.w_in.shape[0])
        ops.check_attention_sizes(H, 1, D, largest=_KERNEL_HEAD_SIZES[-1])

    def state_need(self):
        return PagedKV(1, self.head_dim, self.window)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, D = self.n_heads, self.head_dim
        proj = ctx.buf("latent_proj", (T, self.proj_width), torch.float32)
        ops.linear(x, self.w_in, proj)
        if self.q_latent:
            cq = ctx.buf("latent_cq", (T, self.q_rank), ctx.act_dtype)
            ops.cols_rmsnorm(proj, 0, self.dq_norm, self.norm_eps, cq)
            qf, q0 = ctx.buf("latent_qf", (T, self.q_width), torch.float32), 0
            ops.linear(cq, self.w_uq, qf)
        else:
            qf, q0 = proj, 0
        if self.rot_dim:
            cos, sin = self.position.rotation(ctx)
            ops.latent_rope_append(proj, self.c_col, self.rank, self.rot_dim, self.c_norm, self.norm_eps, cos, sin,
                                   bool(getattr(self.position, "interleaved", False)),
                                   float(getattr(self.position, "magnitude", 1.0)), qf, q0, H, self.dim, ctx, cache)
        elif cache.writes:
            ops.latent_append(proj, self.c_col, self.rank, self.c_norm, self.norm_eps, ctx, cache)
        q = ctx.buf("attn_q", (T, H * D), ctx.act_dtype)
        ops.head_linear(qf, q0, self.w_uk_t, q)
        o = ctx.buf("attn_o", (T, H * D), ctx.act_dtype)
        parts = _decode_parts(H) if (H > 16 and getattr(ctx, "decode_only", False)) else 1
        if parts > 1 and H // parts >= 4:
            rows = _RowsAsParts(ctx, parts)
            with ops.plain_launches():                     # the kernel reads positions early; here a kernel wrote them
                ops.paged_attention(q.view(T * parts, (H // parts) * D), o.view(T * parts, (H // parts) * D), rows,
                                    cache, H // parts, 1, D, self.scale, 0.0, self.window)
        else:
            ops.paged_attention(q, o, ctx, cache, H, 1, D, self.scale, 0.0, self.window)
        v = ctx.buf("latent_v", (T, H * self.vdim), ctx.act_dtype)
        ops.head_linear(o, 0, self.w_uv, v)
        if self.gated:
            gated = ctx.buf("attn_gated", (T, H * self.vdim), ctx.act_dtype)
            ops.head_gate(v, proj, self.g_col, H, self.vdim, self.vdim, gated, ctx)
            v = gated
        y = ctx.buf(self.out_tag, (T, self.width), torch.float32)
        ops.linear(v, self.wo, y)
        return y


register_mixer("latent_attention", LatentAttention)
