"""A plain, slow Nukelix: float64, whole sequences, no cache, one function per mechanism.

Shares nothing with the package.  `cfg` is the dictionary of a config.json, `w` a dictionary name -> tensor.
Notation: W width, H query heads, G key/value heads, d key size, dv value size, r rotated elements of a head.
"""
from __future__ import annotations

import math

import torch

F = torch.float64

# What a 16-bit serving path may round: the inputs of matrix products, queries, keys and values as the attention reads
# them, the attention's weights, the feed-forwards' inner rows.  `ROUND` is applied at those places; the identity by
# default.  `rounded_to_bfloat16()` switches it for a block of code: a yardstick of what 8-bit mantissas alone do.
_EXACT = lambda t: t
ROUND = _EXACT


class rounded_to_bfloat16:
    def __enter__(self):
        global ROUND
        self.saved, ROUND = ROUND, (lambda t: t.to(torch.bfloat16).to(F))

    def __exit__(self, *exc):
        global ROUND
        ROUND = self.saved
        return False


def rms(x, eps: float):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def linear(x, weight, bias=None):
    y = ROUND(x) @ weight.to(F).T
    return y if bias is None else y + bias.to(F)


# ---- rotations ---------------------------------------------------------------------------------------------------

def plain_frequencies(rot: dict):
    r = int(rot["dims"])
    return float(rot["base"]) ** (-2.0 * torch.arange(r // 2, dtype=F) / r)


def wavelength_scaled_frequencies(rot: dict):
    """Frequencies rescaled by wavelength: short waves stay, long waves slow down by `factor`, a linear blend between."""
    f = plain_frequencies(rot)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(f.numel()):
        wave = 2.0 * math.pi / float(f[i])
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = f[i] / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def ramp_scaled_frequencies(rot: dict):
    """(frequencies, factor on cos and sin) of the rescaling by pair index: a ramp between the pairs that make `fast`
    and `slow` turns over `original` positions."""
    f = plain_frequencies(rot)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    r, base = int(rot["dims"]), float(rot["base"])
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), r - 1)
    i = torch.arange(r // 2, dtype=F)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, r: int, interleaved: bool, magnitude: float = 1.0):
    """x [T, heads, n]: the first r elements of every head turned by position * freqs; pairs (2i, 2i+1) when
    `interleaved`, else (i, i + r/2).  cos and sin are multiplied by `magnitude`."""
    if r == 0:
        return x
    ang = positions.to(F)[:, None] * freqs[None, :]
    cos, sin = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:r:2], x[..., 1:r:2]
        out[..., 0:r:2] = u * cos - v * sin
        out[..., 1:r:2] = v * cos + u * sin
    else:
        u, v = x[..., : r // 2], x[..., r // 2: r]
        out[..., : r // 2] = u * cos - v * sin
        out[..., r // 2: r] = v * cos + u * sin
    return out


# ---- attention ----------------------------------------------------------------------------------------------------

def visible(T: int, window: int | None, keep_first: int):
    """[T, T] mask: row i sees column j iff j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m = m & ((i - j < window) | (j < keep_first))
    return m


def attend(q, k, v, scale: float, mask, sink: bool):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Head h reads key/value head h // (H / G).  `sink`: one
    is added to the softmax's denominator (a key of score 0 without a value)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    q, k, v = ROUND(q), ROUND(k), ROUND(v)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        top = s.max(-1, keepdim=True).values
        if sink:
            top = top.clamp(min=0.0)
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True) + (torch.exp(-top) if sink else 0.0)
        out[:, h] = ROUND(e / den) @ v[:, g]
    return out


def gqa_projections(h, w, p: str, m: dict, eps: float):
    """Biased q, k, v of the input rows, q and k normed over the WHOLE projection (all heads at once)."""
    q = linear(h, w[p + "q"], w[p + "q.b"])
    k = linear(h, w[p + "k"], w[p + "k.b"])
    v = linear(h, w[p + "v"], w[p + "v.b"])
    q = rms(q, eps) * w[p + "q.norm"].to(F)
    k = rms(k, eps) * w[p + "k.norm"].to(F)
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    return q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)


def head_gated(o, h, w_gate):
    """o [T, H, dv] times sigmoid(W_g h) [T, H], one number per head."""
    g = torch.sigmoid(linear(h, w_gate))
    return o * g[:, :, None]


def windowed_attention(h, w, p: str, m: dict, eps: float, positions, v_first):
    """The mixer 'attention'.  Returns (result [T, W], this layer's values as they are cached [T, G, dv])."""
    q, k, v = gqa_projections(h, w, p, m, eps)
    rot = m.get("rot")
    if rot:
        f = wavelength_scaled_frequencies(rot)
        q = rotate(q, positions, f, int(rot["dims"]), True)
        k = rotate(k, positions, f, int(rot["dims"]), True)
    if m.get("v_mix") and v_first is not None:
        lam = float(w[p + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    mask_cfg = m.get("mask")
    T = h.shape[0]
    mask = visible(T, int(mask_cfg["size"]), int(mask_cfg.get("keep_first", 0))) if mask_cfg else visible(T, None, 0)
    o = attend(q, k, v, float(m["scale"]), mask, sink=True)
    o = head_gated(o, h, w[p + "g"])
    return linear(o.reshape(T, -1), w[p + "o"]), v


def full_attention(h, w, p: str, m: dict, eps: float, positions):
    """The left half of the mixer 'parallel': causal, ordinary softmax, pairs (i, i + r/2)."""
    q, k, v = gqa_projections(h, w, p, m, eps)
    rot = m.get("rot")
    if rot:
        f = plain_frequencies(rot)
        q = rotate(q, positions, f, int(rot["dims"]), False)
        k = rotate(k, positions, f, int(rot["dims"]), False)
    T = h.shape[0]
    o = attend(q, k, v, float(m["scale"]), visible(T, None, 0), sink=False)
    o = head_gated(o, h, w[p + "g"])
    return linear(o.reshape(T, -1), w[p + "o"])


def memory_walk(q, k, v, gi, gf, state=None):
    """The memory's recurrence alone.  q, k [T, H, d] (q already times d^-1/2), v [T, H, dv], log gates gi, gf [T, H];
    `state` (S [H, d, dv], n [H, d], m [H]) from earlier tokens, or None for the start (zeros; m = 0).
    Returns (o [T, H, dv], state)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    if state is None:
        state = (torch.zeros(H, d, dv, dtype=F), torch.zeros(H, d, dtype=F), torch.zeros(H, dtype=F))
    S, n, m = (x.clone().to(F) for x in state)
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        top = float(m[a])
        for t in range(T):
            new_top = max(float(gf[t, a]) + top, float(gi[t, a]))
            keep, take = math.exp(float(gf[t, a]) + top - new_top), math.exp(float(gi[t, a]) - new_top)
            S[a] = keep * S[a] + take * torch.outer(k[t, a], v[t, a])
            n[a] = keep * n[a] + take * k[t, a]
            top = new_top
            den = max(abs(float(n[a] @ q[t, a])), math.exp(-top)) + 1e-6
            out[t, a] = (S[a].T @ q[t, a]) / den
        m[a] = top
    return out, (S, n, m)


def memory_gates(zi, zf, cap: float):
    """Log input gate and log forget gate from their raw values (biases added)."""
    return cap * torch.tanh(zi / cap), torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))


def matrix_memory(h, w, p: str, m: dict, eps: float):
    """The right half of the mixer 'parallel': a d x dv memory per head with exponential gates kept stable by a running
    maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (linear(h, w[p + "q"]) * d ** -0.5).view(T, H, d)
    k = linear(h, w[p + "k"]).view(T, H, d)
    v = linear(h, w[p + "v"]).view(T, H, dv)
    gi, gf = memory_gates(linear(h, w[p + "i"], w[p + "i.b"]), linear(h, w[p + "f"], w[p + "f.b"]), cap)
    out, _ = memory_walk(q, k, v, gi, gf)
    o = rms(out, eps).reshape(T, H * dv) * w[p + "norm"].to(F)
    o = o * torch.sigmoid(linear(h, w[p + "g"]))
    return linear(o, w[p + "o"])


def parallel_mixers(h, w, p: str, m: dict, eps: float, positions):
    left = full_attention(h, w, p + "left.", m["left"], eps, positions)
    right = matrix_memory(h, w, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def latent_attention(h, w, p: str, m: dict, eps: float, positions):
    """Queries through a normed latent; keys and values from a normed latent c of every token plus one rotated key
    part that all heads share."""
    T = h.shape[0]
    H, d, r, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms(linear(h, w[p + "dq"]), eps) * w[p + "dq.norm"].to(F)
    q = linear(cq, w[p + "uq"]).view(T, H, d + r)
    down = linear(h, w[p + "dkv"])
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"].to(F)
    k_rot = down[:, rank:].view(T, 1, r)
    k_flat = linear(c, w[p + "uk"]).view(T, H, d)
    v = linear(c, w[p + "uv"]).view(T, H, dv)
    if m.get("rot"):
        f, mag = ramp_scaled_frequencies(dict(m["rot"]))
        q_rot = rotate(q[..., d:], positions, f, r, True, mag)
        k_rot = rotate(k_rot, positions, f, r, True, mag)
    else:
        q_rot = q[..., d:]
    if ROUND is not _EXACT:                                  # a 16-bit path caches c alone and rounds in the latent space
        o = latent_space_attention(q[..., :d], q_rot, c, k_rot, w, p, m)
    else:
        qq = torch.cat([q[..., :d], q_rot], dim=-1)
        kk = torch.cat([k_flat, k_rot.expand(T, H, r)], dim=-1)
        o = attend(qq, kk, v, float(m["scale"]), visible(T, None, 0), sink=False)
    o = head_gated(o, h, w[p + "g"])
    return linear(o.reshape(T, -1), w[p + "o"])


def latent_space_attention(q_flat, q_rot, c, k_rot, w, p: str, m: dict):
    """The same attention with every query taken into the latent space, q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, and the
    values' map applied after the weighted sum, sum_j a_j W_uv,h c_j = W_uv,h sum_j a_j c_j: equal in exact arithmetic; a
    16-bit path that caches c alone rounds here (the queries in the latent space, c, the weighted sums of c)."""
    T, H, d = q_flat.shape
    rank, dv, r = c.shape[-1], int(m["vdim"]), q_rot.shape[-1]
    uk = w[p + "uk"].to(F).view(H, d, rank)
    uv = w[p + "uv"].to(F).view(H, dv, rank)
    qa = torch.einsum("thd,hdr->thr", ROUND(q_flat), uk)
    qq = torch.cat([qa, q_rot], dim=-1)
    kk = torch.cat([c, k_rot[:, 0]], dim=-1)[:, None, :]
    vv = torch.cat([c, torch.zeros(T, r, dtype=F)], dim=-1)[:, None, :]
    o = attend(qq, kk, vv, float(m["scale"]), visible(T, None, 0), sink=False)
    return ROUND(torch.einsum("thr,hvr->thv", ROUND(o[..., :rank]), uv))


# ---- feed-forward --------------------------------------------------------------------------------------------------

def gated_expert(x, w, p: str):
    g, u = linear(x, w[p + "gate"]), linear(x, w[p + "up"])
    return linear(g * torch.sigmoid(g) * u, w[p + "down"])


def route(h, w_router, top: int):
    """(ids [T, top], weights [T, top]): the experts with the largest sigmoid scores and those scores themselves."""
    s = torch.sigmoid(ROUND(h) @ w_router.to(F).T)
    best = torch.topk(s, top, dim=-1)
    return best.indices, best.values


def mixture(h, w, p: str, f: dict):
    """sum over the chosen experts of expert(weight * h), plus the shared expert."""
    ids, wts = route(h, w[p + "router"], int(f["router"]["top"]))
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for c in range(ids.shape[1]):
        for e in ids[:, c].unique().tolist():
            rows = (ids[:, c] == e).nonzero().flatten()
            out[rows] += gated_expert(wts[rows, c:c + 1] * h[rows], w, f"{p}e{e}.")
    if f.get("shared"):
        out = out + gated_expert(h, w, p + "shared.")
    return out


# ---- the model -----------------------------------------------------------------------------------------------------

def residuals(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """The residual stream after every layer [layers, T, W] of one sequence."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = w["embed"].to(F)[tokens]
    v_first, out = None, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            a, v = windowed_attention(x, w, p + "mix.", m, eps, positions, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif layer["type"] == "parallel":
            a = parallel_mixers(x, w, p + "mix.", m, eps, positions)
        elif layer["type"] == "latent_attention":
            a = latent_attention(x, w, p + "mix.", m, eps, positions)
        else:
            raise ValueError(layer["type"])
        x = x + rms(a, eps) * w[p + "norm1"].to(F)
        if layer.get("mlp"):
            x = x + rms(mixture(x, w, p + "mlp.", layer["mlp"]), eps) * w[p + "norm2"].to(F)
        out.append(x)
    return torch.stack(out)


def logits_of(cfg: dict, w: dict, x) -> torch.Tensor:
    h = rms(x, float(cfg["norm"]["eps"])) * w["final.norm"].to(F)
    z = linear(h, w["embed"])
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap > 0 else z


def forward(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """Logits [T, vocab] of one sequence."""
    return logits_of(cfg, w, residuals(cfg, w, tokens)[-1])
