"""Pimodra put together from parts.

A Pimodra model is a list of blocks with a norm before and after each sublayer (`parts.SandwichBlock`), all norms being
RMS norms in groups (`parts.GroupRmsNorm`).  The mixer is grouped-query attention with rotated, unit-norm queries and
keys, a sliding window, softmax weights mixed across heads and an element-wise output gate (`parts.TalkingAttention`);
the rotation's slow pairs are stretched (`parts.Rope(yarn=...)`).  The feed-forward is an ungated one whose activation
norms the powers of its input (`parts.PolyNormFfn`), a mixture of silu-gated experts with softmax scores whose winners
keep their scores (`parts.RoutedExperts`), or absent.  A stretch of layers may run several times in a row with the same
weights: every run is a call of the model's schedule with a cache slot of its own, and the first call of each pass adds
that pass's row of `loop.step` to the residual (`LayerCall.shift`).  The output is a norm and the embedding table itself.
Tensor names are those of a Pimodra safetensors file: `embed`, `loop.step`, `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.mix.q|k|v|g|o|talk`, `l<i>.mlp.up|down|act` or `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`, `final.norm`.
"""
from __future__ import annotations

import torch

from ..config.pimodra import PimodraConfig
from ..parts import (DecoderModel, Embedding, GroupRmsNorm, LayerCall, LmHead, PolyNormFfn, Rope, RoutedExperts, SandwichBlock,
                     TalkingAttention)
from ..weights.store import TensorSpec, WeightStore

MATRIX_STD = 0.02


def _layer_specs(cfg: PimodraConfig, i: int) -> list[TensorSpec]:
    l, W, p = cfg.layers[i], cfg.width, f"l{i}."
    m = l.mixer
    out = [TensorSpec(p + "norm1", (W,), 1.0, "norm"), TensorSpec(p + "norm1b", (W,), 1.0, "norm"),
           TensorSpec(p + "mix.q", (m.heads * m.dim, W), MATRIX_STD), TensorSpec(p + "mix.k", (m.kv_heads * m.dim, W), MATRIX_STD),
           TensorSpec(p + "mix.v", (m.kv_heads * m.vdim, W), MATRIX_STD), TensorSpec(p + "mix.talk", (m.heads, m.heads), 0.5, "norm"),
           TensorSpec(p + "mix.g", (m.heads * m.vdim, W), MATRIX_STD), TensorSpec(p + "mix.o", (W, m.heads * m.vdim), MATRIX_STD)]
    f = l.mlp
    if f is not None:
        out += [TensorSpec(p + "norm2", (W,), 1.0, "norm"), TensorSpec(p + "norm2b", (W,), 1.0, "norm")]
        if f.kind == "dense":
            out += [TensorSpec(p + "mlp.up", (f.ff, W), MATRIX_STD), TensorSpec(p + "mlp.down", (W, f.ff), MATRIX_STD),
                    TensorSpec(p + "mlp.act", (4,), 0.5, "norm")]
        else:
            for e in range(f.experts):
                q = f"{p}mlp.e{e}."
                out += [TensorSpec(q + "gate", (f.ff, W), MATRIX_STD), TensorSpec(q + "up", (f.ff, W), MATRIX_STD),
                        TensorSpec(q + "down", (W, f.ff), MATRIX_STD)]
            out.append(TensorSpec(p + "mlp.router", (f.experts, W), MATRIX_STD))
    return out


def tensor_specs(cfg: PimodraConfig) -> list[TensorSpec]:
    """Every tensor a Pimodra file holds for `cfg`, with the spread random weights are drawn with."""
    specs = [TensorSpec("embed", (cfg.vocab, cfg.width), MATRIX_STD)]
    if cfg.loop is not None:
        specs.append(TensorSpec("loop.step", (cfg.loop.times, cfg.width), MATRIX_STD))
    for i in range(len(cfg.layers)):
        specs += _layer_specs(cfg, i)
    specs.append(TensorSpec("final.norm", (cfg.width,), 1.0, "norm"))
    return specs


def _stack(parts: list[torch.Tensor]) -> torch.Tensor:
    if any(p.numel() == 0 for p in parts) or len({p.dtype for p in parts}) != 1:
        return torch.empty(0)                       # a fault already recorded by the store
    return torch.cat(parts, dim=0).contiguous()


def _mixer(cfg: PimodraConfig, w: WeightStore, i: int, ropes: dict) -> TalkingAttention:
    m, W, p = cfg.layers[i].mixer, cfg.width, f"l{i}.mix."
    rows = (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim), ("g", m.heads * m.vdim))
    w_in = _stack([w.take(p + n, (r, W)) for n, r in rows])             # [q | k | v | gate] rows
    w.release(*[p + n for n, _ in rows])
    rope = None
    if m.rot is not None:
        # layers with the same rotary constants share one table per step
        rope = ropes.get((m.dim, m.rot))
        if rope is None:
            rope = ropes[(m.dim, m.rot)] = Rope(m.dim, m.rot.base, w.device, m.rot.dims, yarn=m.rot.yarn_dict())
    return TalkingAttention(w_in, w.take(p + "o", (W, m.heads * m.vdim)), n_heads=m.heads, n_kv_heads=m.kv_heads, key_dim=m.dim,
                            value_dim=m.vdim, scale=m.scale, window=m.window, position=rope,
                            mix=w.take(p + "talk", (m.heads, m.heads)), unit_norm=True, norm_eps=cfg.norm_eps, gated=True)


def _feed_forward(cfg: PimodraConfig, w: WeightStore, i: int):
    f, W, p = cfg.layers[i].mlp, cfg.width, f"l{i}.mlp."
    if f.kind == "dense":
        return PolyNormFfn(w.take(p + "up", (f.ff, W)), w.take(p + "down", (W, f.ff)), w.take(p + "act", (4,)), cfg.norm_eps)
    gus, downs = [], []
    for e in range(f.experts):
        q = f"{p}e{e}."
        gus.append(_stack([w.take(q + "gate", (f.ff, W)), w.take(q + "up", (f.ff, W))]))
        w.release(q + "gate", q + "up")
        downs.append(w.take(q + "down", (W, f.ff)))
    router = w.take(p + "router", (f.experts, W))
    if w.faulty:
        w.finish()
    w_gate_up, w_down = torch.stack(gus).contiguous(), torch.stack(downs).contiguous()
    w.release(*[f"{p}e{e}.down" for e in range(f.experts)])
    return RoutedExperts(router, None, w_gate_up, w_down, top=f.top, scale=1.0, limit=0.0, groups=f.groups, keep=f.keep,
                         score="softmax", group_rank="best", normalize=False, activation="silu")


def build(cfg: PimodraConfig, w: WeightStore) -> DecoderModel:
    W = cfg.width
    table = w.take("embed", (cfg.vocab, W))
    steps = w.take("loop.step", (cfg.loop.times, W)) if cfg.loop is not None else None
    if w.faulty:
        w.finish()

    def norm(name: str) -> GroupRmsNorm:
        return GroupRmsNorm(w.take(name, (W,)), cfg.norm_eps, cfg.norm_groups)

    blocks, ropes = [], {}
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        mixer = _mixer(cfg, w, i, ropes)
        norm1, norm1b = norm(p + "norm1"), norm(p + "norm1b")
        ffn = norm2 = norm2b = None
        if l.mlp is not None:
            ffn = _feed_forward(cfg, w, i)
            norm2, norm2b = norm(p + "norm2"), norm(p + "norm2b")
        if w.faulty:
            w.finish()
        blocks.append(SandwichBlock(norm1, mixer, norm1b, norm2, ffn, norm2b))
    final_norm = norm("final.norm")
    w.finish()
    # one call per layer run, each with a cache slot of its own; the first call of a pass adds the pass's row
    schedule = []
    for slot, (i, t) in enumerate(cfg.layer_runs()):
        first_of_pass = t is not None and i == cfg.loop.start
        schedule.append(LayerCall(i, slot, shift=steps[t].contiguous() if first_of_pass else None))
    return DecoderModel(Embedding(table), blocks, LmHead(final_norm, table), schedule, name=cfg.architecture)
