"""Nukelix put together from parts.

A Nukelix model is a list of blocks whose sublayers read the residual stream itself and whose results are normed before
they join it: `x += norm1(mixer(x)); x += norm2(ff(x))` (`parts.SandwichBlock` with `parts.NoNorm` in the places of the
norms before the sublayers).  A layer's mixer is one of
  attention         grouped-query attention with biased projections, q and k normed over the whole projection, interleaved
                    rotary pairs with frequencies rescaled by wavelength, a sliding window that keeps the first tokens, one
                    added to the softmax's denominator, values mixed with those of the first such layer, a gate per head
                    (`parts.RowNormAttention`);
  parallel          two mixers side by side on the same input (`parts.SideBySide`): the same attention without window,
                    sink or mixing and with pairs (i, i + dims/2), beside a matrix memory with exponential gates
                    (`parts.MatrixMemory`);
  latent_attention  attention over a cached latent with queries through a latent of their own, one rotated key part that
                    all heads share (interleaved pairs, frequencies stretched by pair index) and a gate per head
                    (`parts.LatentAttention`).
The feed-forward is a mixture of silu-gated experts with sigmoid scores whose winners' scores multiply the experts'
inputs, plus a shared expert (`parts.RoutedExperts`), or absent.  The output is a norm, the embedding table itself and a
cap on the logits.
Tensor names are those of a Nukelix safetensors file: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.*` (attention:
q|k|v (+ `.b`), q.norm, k.norm, vmix, g, o; parallel: the same under `left.` and q|k|v|g|o|norm|i|f (+ `i.b`, `f.b`) under
`right.`; latent: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o), `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`,
`l<i>.mlp.shared.gate|up|down`, `final.norm`.
"""
from __future__ import annotations

import torch

from ..config.nukelix import ATTENTION, LATENT, PARALLEL, AttentionSpec, NukelixConfig
from ..parts import (DecoderModel, Embedding, GatedFfn, LatentAttention, LmHead, MatrixMemory, NoNorm, RmsNorm, Rope,
                     RoutedExperts, RowNormAttention, SandwichBlock, SideBySide)
from ..weights.store import TensorSpec, WeightStore

MATRIX_STD = 0.02


def _attention_specs(m: AttentionSpec, W: int, p: str, v_mix: bool) -> list[TensorSpec]:
    nq, nk, nv = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
    out = [TensorSpec(p + "q", (nq, W), MATRIX_STD), TensorSpec(p + "q.b", (nq,), MATRIX_STD),
           TensorSpec(p + "k", (nk, W), MATRIX_STD), TensorSpec(p + "k.b", (nk,), MATRIX_STD),
           TensorSpec(p + "v", (nv, W), MATRIX_STD), TensorSpec(p + "v.b", (nv,), MATRIX_STD),
           TensorSpec(p + "q.norm", (nq,), 1.0, "norm"), TensorSpec(p + "k.norm", (nk,), 1.0, "norm")]
    if v_mix:
        out.append(TensorSpec(p + "vmix", (), 0.3, "norm"))
    return out + [TensorSpec(p + "g", (m.heads, W), MATRIX_STD), TensorSpec(p + "o", (W, m.heads * m.vdim), MATRIX_STD)]


def _expert_specs(p: str, ff: int, W: int) -> list[TensorSpec]:
    return [TensorSpec(p + "gate", (ff, W), MATRIX_STD), TensorSpec(p + "up", (ff, W), MATRIX_STD),
            TensorSpec(p + "down", (W, ff), MATRIX_STD)]


def _layer_specs(cfg: NukelixConfig, i: int) -> list[TensorSpec]:
    l, W, p = cfg.layers[i], cfg.width, f"l{i}."
    m = l.mixer
    out = [TensorSpec(p + "norm1", (W,), 1.0, "norm")]
    if l.mlp is not None:
        out.append(TensorSpec(p + "norm2", (W,), 1.0, "norm"))
    if l.type == ATTENTION:
        out += _attention_specs(m, W, p + "mix.", m.v_mix)
    elif l.type == PARALLEL:
        out += _attention_specs(m.left, W, p + "mix.left.", False)
        r, q = m.right, p + "mix.right."
        out += [TensorSpec(q + "q", (r.heads * r.dim, W), MATRIX_STD), TensorSpec(q + "k", (r.heads * r.dim, W), MATRIX_STD),
                TensorSpec(q + "v", (r.heads * r.vdim, W), MATRIX_STD), TensorSpec(q + "g", (r.heads * r.vdim, W), MATRIX_STD),
                TensorSpec(q + "o", (W, r.heads * r.vdim), MATRIX_STD), TensorSpec(q + "norm", (r.heads * r.vdim,), 1.0, "norm"),
                TensorSpec(q + "i", (r.heads, W), MATRIX_STD), TensorSpec(q + "i.b", (r.heads,), MATRIX_STD),
                TensorSpec(q + "f", (r.heads, W), MATRIX_STD), TensorSpec(q + "f.b", (r.heads,), 1.0, "norm")]
    else:
        q = p + "mix."
        out += [TensorSpec(q + "dq", (m.q_rank, W), MATRIX_STD), TensorSpec(q + "dq.norm", (m.q_rank,), 1.0, "norm"),
                TensorSpec(q + "uq", (m.heads * (m.dim + m.rot_dim), m.q_rank), MATRIX_STD),
                TensorSpec(q + "dkv", (m.kv_rank + m.rot_dim, W), MATRIX_STD), TensorSpec(q + "dkv.norm", (m.kv_rank,), 1.0, "norm"),
                TensorSpec(q + "uk", (m.heads * m.dim, m.kv_rank), MATRIX_STD), TensorSpec(q + "uv", (m.heads * m.vdim, m.kv_rank), MATRIX_STD),
                TensorSpec(q + "g", (m.heads, W), MATRIX_STD), TensorSpec(q + "o", (W, m.heads * m.vdim), MATRIX_STD)]
    f = l.mlp
    if f is not None:
        for e in range(f.experts):
            out += _expert_specs(f"{p}mlp.e{e}.", f.ff, W)
        out.append(TensorSpec(p + "mlp.router", (f.experts, W), MATRIX_STD))
        if f.shared_ff:
            out += _expert_specs(p + "mlp.shared.", f.shared_ff, W)
    return out


def tensor_specs(cfg: NukelixConfig) -> list[TensorSpec]:
    """Every tensor a Nukelix file holds for `cfg`, with the spread random weights are drawn with."""
    specs = [TensorSpec("embed", (cfg.vocab, cfg.width), MATRIX_STD)]
    for i in range(len(cfg.layers)):
        specs += _layer_specs(cfg, i)
    specs.append(TensorSpec("final.norm", (cfg.width,), 1.0, "norm"))
    return specs


def _stack(parts: list[torch.Tensor]) -> torch.Tensor:
    if any(p.numel() == 0 for p in parts) or len({p.dtype for p in parts}) != 1:
        return torch.empty(0)                       # a fault already recorded by the store
    return torch.cat(parts, dim=0).contiguous()


def _rope(ropes: dict, key: tuple, make):
    # mixers with the same rotary constants share one table per step
    if key not in ropes:
        ropes[key] = make()
    return ropes[key]


def _attention(cfg: NukelixConfig, w: WeightStore, m: AttentionSpec, p: str, ropes: dict, *, windowed: bool,
               v_mix: str | None) -> RowNormAttention:
    W = cfg.width
    nq, nk, nv = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
    rows = (("q", nq), ("k", nk), ("v", nv), ("g", m.heads))
    w_in = _stack([w.take(p + n, (r, W)) for n, r in rows])                 # [q | k | v | gate] rows
    bias = _stack([w.take(p + n + ".b", (r,)) for n, r in rows[:3]])
    w.release(*[p + n for n, _ in rows], *[p + n + ".b" for n, _ in rows[:3]])
    rope = None
    if m.rot is not None:
        if windowed:                                # interleaved pairs, frequencies rescaled by wavelength
            rope = _rope(ropes, ("w", m.dim, m.rot), lambda: Rope(m.dim, m.rot.base, w.device, m.rot.dims, interleaved=True,
                                                                  scaling=m.rot.wavelength_dict()))
        else:                                       # pairs (i, i + dims/2), plain frequencies
            rope = _rope(ropes, ("h", m.dim, m.rot), lambda: Rope(m.dim, m.rot.base, w.device, m.rot.dims))
    lam = w.take(p + "vmix", ()) if windowed and m.v_mix else None
    return RowNormAttention(w_in, w.take(p + "o", (W, m.heads * m.vdim)), n_heads=m.heads, n_kv_heads=m.kv_heads,
                            key_dim=m.dim, value_dim=m.vdim, scale=m.scale, window=m.window if windowed else None,
                            keep_first=m.keep_first if windowed else 0, sink=windowed, position=rope,
                            bias=bias if bias.numel() else None, q_norm=w.take(p + "q.norm", (nq,)),
                            k_norm=w.take(p + "k.norm", (nk,)), norm_eps=cfg.norm_eps, gated=True, v_mix=v_mix,
                            v_mix_weight=lam if v_mix == "mix" else None)


def _memory(cfg: NukelixConfig, w: WeightStore, r, p: str) -> MatrixMemory:
    W = cfg.width
    rows = (("q", r.heads * r.dim), ("k", r.heads * r.dim), ("v", r.heads * r.vdim), ("g", r.heads * r.vdim),
            ("i", r.heads), ("f", r.heads))
    w_in = _stack([w.take(p + n, (n_rows, W)) for n, n_rows in rows])      # [q | k | v | gate | input gate | forget gate]
    w.release(*[p + n for n, _ in rows])
    return MatrixMemory(w_in, w.take(p + "o", (W, r.heads * r.vdim)), w.take(p + "i.b", (r.heads,)),
                        w.take(p + "f.b", (r.heads,)), w.take(p + "norm", (r.heads * r.vdim,)), heads=r.heads, dim=r.dim,
                        vdim=r.vdim, gate_cap=r.gate_cap, norm_eps=cfg.norm_eps)


def _latent(cfg: NukelixConfig, w: WeightStore, m, p: str, ropes: dict) -> LatentAttention:
    W = cfg.width
    rope = None
    if m.rot is not None:
        rope = _rope(ropes, ("l", m.rot_dim, m.rot), lambda: Rope(m.rot_dim, m.rot.base, w.device, m.rot_dim, interleaved=True,
                                                                  yarn=m.rot.ramp_dict()))
    mixer = LatentAttention(w.take(p + "uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),
                            w.take(p + "dkv", (m.kv_rank + m.rot_dim, W)), w.take(p + "dkv.norm", (m.kv_rank,)),
                            w.take(p + "uk", (m.heads * m.dim, m.kv_rank)), w.take(p + "uv", (m.heads * m.vdim, m.kv_rank)),
                            w.take(p + "o", (W, m.heads * m.vdim)), n_heads=m.heads, dim=m.dim, vdim=m.vdim, rank=m.kv_rank,
                            scale=m.scale, norm_eps=cfg.norm_eps, w_dq=w.take(p + "dq", (m.q_rank, W)),
                            dq_norm=w.take(p + "dq.norm", (m.q_rank,)), rot_dim=m.rot_dim, position=rope,
                            w_gate=w.take(p + "g", (m.heads, W)))
    w.release(p + "dq", p + "dkv", p + "g", p + "uk", p + "uv")
    return mixer


def _gated(w: WeightStore, p: str, ff: int, W: int):
    gu = _stack([w.take(p + "gate", (ff, W)), w.take(p + "up", (ff, W))])
    w.release(p + "gate", p + "up")
    return gu, w.take(p + "down", (W, ff))


def _feed_forward(cfg: NukelixConfig, w: WeightStore, i: int) -> RoutedExperts:
    f, W, p = cfg.layers[i].mlp, cfg.width, f"l{i}.mlp."
    gus, downs = [], []
    for e in range(f.experts):
        gu, down = _gated(w, f"{p}e{e}.", f.ff, W)
        gus.append(gu)
        downs.append(down)
    router = w.take(p + "router", (f.experts, W))
    shared = None
    if f.shared_ff:
        gu, down = _gated(w, p + "shared.", f.shared_ff, W)
        if gu.numel() and down.numel():
            shared = GatedFfn(gu, down, "silu")
    if w.faulty:
        w.finish()
    w_gate_up, w_down = torch.stack(gus).contiguous(), torch.stack(downs).contiguous()
    w.release(*[f"{p}e{e}.down" for e in range(f.experts)])
    return RoutedExperts(router, None, w_gate_up, w_down, top=f.top, scale=1.0, limit=0.0, shared=shared, score="sigmoid",
                         group_rank="best", normalize=False, activation="silu", weight_on="input")


def build(cfg: NukelixConfig, w: WeightStore) -> DecoderModel:
    W = cfg.width
    table = w.take("embed", (cfg.vocab, W))
    if w.faulty:
        w.finish()
    mixed = cfg.v_mix_layers()
    blocks, ropes = [], {}
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.type == ATTENTION:
            role = None if i not in mixed else ("first" if i == mixed[0] else "mix")
            mixer = _attention(cfg, w, l.mixer, p + "mix.", ropes, windowed=True, v_mix=role)
        elif l.type == PARALLEL:
            left = _attention(cfg, w, l.mixer.left, p + "mix.left.", ropes, windowed=False, v_mix=None)
            right = _memory(cfg, w, l.mixer.right, p + "mix.right.")
            mixer = SideBySide(left, right, l.mixer.left_scale, l.mixer.right_scale)
        else:
            mixer = _latent(cfg, w, l.mixer, p + "mix.", ropes)
        norm1 = RmsNorm(w.take(p + "norm1", (W,)), cfg.norm_eps)
        ffn = norm2 = None
        if l.mlp is not None:
            ffn = _feed_forward(cfg, w, i)
            norm2 = RmsNorm(w.take(p + "norm2", (W,)), cfg.norm_eps)
        if w.faulty:
            w.finish()
        blocks.append(SandwichBlock(NoNorm(W), mixer, norm1, NoNorm(W) if ffn is not None else None, ffn, norm2))
    final_norm = RmsNorm(w.take("final.norm", (W,)), cfg.norm_eps)
    w.finish()
    return DecoderModel(Embedding(table), blocks, LmHead(final_norm, table, cfg.logit_softcap), name=cfg.architecture)
