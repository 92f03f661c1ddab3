"""A plain, slow Pimodra: float64, whole sequences, no cache, one function per mechanism.

Shares nothing with the package.  `cfg` is the dictionary of a config.json, `w` a dictionary name -> tensor.
Notation: W width, H query heads, G key/value heads, d key size, dv value size, r rotated elements of a head.
"""
from __future__ import annotations

import math

import torch

F = torch.float64

# What a 16-bit serving path may round: the inputs of matrix products (normed rows, the heads after the attention, the
# feed-forward's inner rows), queries, keys and values as the attention reads them, and the attention's weights.  `ROUND`
# is applied at those places; the identity by default.  `rounded_to_bfloat16()` switches it for a block of code, which
# gives a yardstick of how far 8-bit mantissas alone move a model's logits.
ROUND = lambda t: t


class rounded_to_bfloat16:
    def __enter__(self):
        global ROUND
        self.saved, ROUND = ROUND, (lambda t: t.to(torch.bfloat16).to(F))

    def __exit__(self, *exc):
        global ROUND
        ROUND = self.saved
        return False


def group_norm(x, weight, eps: float, groups: int):
    """x [T, W] cut into `groups` equal consecutive parts; each part is divided by sqrt(mean(part^2) + eps); then * weight."""
    T, W = x.shape
    p = x.reshape(T, groups, W // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(T, W) * weight.to(F)


def yarn_frequencies(rot: dict):
    """(frequencies [r/2], factor on cos and sin) of a rotation whose `scaling` stretches the slow pairs."""
    r, base = int(rot["dims"]), float(rot["base"])
    half = r // 2
    i = torch.arange(half, dtype=F)
    f = base ** (-2.0 * i / r)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):                      # the pair index whose wavelength makes `turns` turns over `original` positions
        return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), r - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict | None):
    """x [T, heads, d]: the first r elements of every head turned in pairs (i, i + r/2) by position * frequency_i."""
    if not rot:
        return x
    f, mag = yarn_frequencies(rot)
    r = int(rot["dims"])
    half = r // 2
    ang = positions.to(F)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    a, b = x[..., :half], x[..., half:r]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., r:]], dim=-1)


def unit_rms(x, eps: float):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def talking_attention(h, m: dict, w: dict, p: str, eps: float, positions=None):
    """The attention mixer on the normed rows h [T, W] of ONE sequence; m = the layer's `mixer` dictionary, p = 'l<i>.mix.'."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].to(F).T).reshape(T, H, d)
    k = (h @ w[p + "k"].to(F).T).reshape(T, G, d)
    v = (h @ w[p + "v"].to(F).T).reshape(T, G, dv)
    q = ROUND(unit_rms(rotate(q, pos, m.get("rot")), eps))
    k = ROUND(unit_rms(rotate(k, pos, m.get("rot")), eps))
    v = ROUND(v)
    per = H // G
    kv_of = torch.arange(H) // per
    s = torch.einsum("ihd,jhd->hij", q, k[:, kv_of, :]) * float(m["scale"])
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i)
    size = (m.get("mask") or {}).get("size")
    if size:
        seen = seen & (i - j < int(size))
    s = s.masked_fill(~seen[None], float("-inf"))
    a = ROUND(torch.softmax(s, dim=-1))                            # [H, T, T], each head's own weights
    a = torch.einsum("hg,gij->hij", w[p + "talk"].to(F), a)        # heads' weights mixed after the softmax
    o = torch.einsum("hij,jhv->ihv", a, v[:, kv_of, :]).reshape(T, H * dv)
    o = ROUND(ROUND(o) * torch.sigmoid(h @ w[p + "g"].to(F).T))
    return o @ w[p + "o"].to(F).T


def poly_norm(z, coef, eps: float):
    """a N(z) + b N(z^2) + c N(z^3) + e, N = division of a row by its root mean square."""
    a, b, c, e = (float(x) for x in coef.to(F))
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ffn(h, w: dict, p: str, eps: float):
    return ROUND(poly_norm(h @ w[p + "up"].to(F).T, w[p + "act"], eps)) @ w[p + "down"].to(F).T


def route(z, experts: int, top: int, groups: int, keep: int):
    """(ids [T, top], weights [T, top]) from router logits z [T, E]: softmax scores; a group of neighbours scores its
    best member; experts outside the `keep` best groups cannot win; the winners keep their scores as weights."""
    s = torch.softmax(z, dim=-1)
    T = z.shape[0]
    allowed = torch.ones_like(s, dtype=torch.bool)
    if groups > 1:
        per = experts // groups
        gs = s.reshape(T, groups, per).max(-1).values
        best = gs.topk(keep, dim=-1).indices
        gmask = torch.zeros(T, groups, dtype=torch.bool)
        gmask.scatter_(1, best, True)
        allowed = gmask[:, :, None].expand(T, groups, per).reshape(T, experts)
    ids = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    return ids, s.gather(1, ids)


def moe_ffn(h, f: dict, w: dict, p: str, router_input=None):
    """A mixture of gated experts with silu; `router_input` lets a caller route on rounded rows."""
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {}
    hr = h if router_input is None else router_input
    ids, wts = route(hr @ w[p + "router"].to(F).T, E, top, int(g.get("count", 1)), int(g.get("keep", 1)))
    y = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(ids[t, c])
            gate, up = w[f"{p}e{e}.gate"].to(F) @ h[t], w[f"{p}e{e}.up"].to(F) @ h[t]
            y[t] += wts[t, c] * (w[f"{p}e{e}.down"].to(F) @ ROUND(gate * torch.sigmoid(gate) * up))
    return y


def layer(x, cfg: dict, w: dict, i: int):
    l, p = cfg["layers"][i], f"l{i}."
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    a = talking_attention(ROUND(group_norm(x, w[p + "norm1"], eps, groups)), l["mixer"], w, p + "mix.", eps)
    x = x + group_norm(a, w[p + "norm1b"], eps, groups)
    f = l.get("mlp")
    if f is None:
        return x
    h = ROUND(group_norm(x, w[p + "norm2"], eps, groups))
    y = dense_ffn(h, w, p + "mlp.", eps) if f.get("kind", "dense") == "dense" else moe_ffn(h, f, w, p + "mlp.")
    return x + group_norm(y, w[p + "norm2b"], eps, groups)


def layer_runs(cfg: dict):
    """[(layer index, pass number or None)] in running order."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg: dict, w: dict, tokens, keep_layers: bool = False):
    """Logits [T, vocab] of one sequence; with `keep_layers` also the residual after every layer run."""
    x = w["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    lp = cfg.get("loop")
    start = int(lp["start"]) if lp else -1
    after = []
    for i, t in layer_runs(cfg):
        if t is not None and i == start:
            x = x + w["loop.step"].to(F)[t]
        x = layer(x, cfg, w, i)
        after.append(x)
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    logits = ROUND(group_norm(x, w["final.norm"], eps, groups)) @ w["embed"].to(F).T
    return (logits, torch.stack(after)) if keep_layers else logits
