"""Rotary position encoding.

For a token at position p and pair index i < r/2 (r = rotary dims, by default the whole
head): angle = p * base^(-2i/r); the pair is (x_i, x_{i+r/2}) ("NeoX" pairing,
reference: crates/kf-backend-cpu/src/rope.rs:18-37,57-108 and gemma2.rs:19):
  x'_i       = x_i cos - x_{i+r/2} sin
  x'_{i+r/2} = x_i sin + x_{i+r/2} cos
The inverse frequencies are computed once in 64-bit and rounded to 32-bit; the angle,
its cosine and sine are 32-bit and are tabulated once per step for all layers that
share this part.

Two options for other models.  `interleaved`: the pair is (x_{2i}, x_{2i+1}) instead; the table is the same, and
the mixer's kernel reads `interleaved` to know which elements a table column turns.  `scaling`
(factor, low, high, original): the frequency rescaling for long contexts in the manner of Llama 3.1, by wavelength
l = 2 pi / f: f is kept where l < original / high, divided by factor where l > original / low, and blended
linearly in between with s = (original / l - low) / (high - low): (1 - s) f / factor + s f.
`yarn` (factor, original, fast, slow): the rescaling by pair index instead.  With p(t) = r ln(original / (2 pi t)) /
(2 ln base), the pair whose wave makes t turns over `original` positions, lo = max(floor(p(fast)), 0),
hi = min(ceil(p(slow)), r - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):
f_i <- ramp_i f_i / factor + (1 - ramp_i) f_i, and `magnitude` = 0.1 ln(factor) + 1 is the factor a consumer multiplies
cos and sin with (1 for every other rotation; the table itself stays cos and sin).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding, register_position


class Rope(PositionEncoding):
    def __init__(self, head_dim: int, base: float, device, rotary_dims: int | None = None, *,
                 interleaved: bool = False, scaling: dict | None = None, yarn: dict | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dims = int(rotary_dims if rotary_dims is not None else head_dim)
        if self.rotary_dims % 2 or self.rotary_dims > self.head_dim:
            raise ValueError(f"rotary_dims {self.rotary_dims} must be even and at most head_dim {self.head_dim}")
        self.base = float(base)
        half = self.rotary_dims // 2
        idx = torch.arange(half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * idx / self.rotary_dims)
        self.interleaved = bool(interleaved)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling:
            factor, low, high = (float(self.scaling[k]) for k in ("factor", "low", "high"))
            original = float(self.scaling["original"])
            if not (factor > 0 and high > low and original > 0):
                raise ValueError(f"rotary scaling needs factor > 0, high > low and original > 0, found {self.scaling}")
            wavelength = 2.0 * math.pi / inv
            blend = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
            mixed = (1.0 - blend) * inv / factor + blend * inv
            inv = torch.where(wavelength < original / high, inv, torch.where(wavelength > original / low, inv / factor, mixed))
        self.yarn = dict(yarn) if yarn else None
        self.magnitude = 1.0
        if self.yarn:
            factor, original = float(self.yarn["factor"]), float(self.yarn["original"])
            fast, slow = float(self.yarn["fast"]), float(self.yarn["slow"])
            if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and self.base > 1):
                raise ValueError(f"yarn scaling needs positive factor, original, fast and slow, found {self.yarn}")

            def pair_of(turns: float) -> float:
                return self.rotary_dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

            lo = max(math.floor(pair_of(fast)), 0)
            hi = min(math.ceil(pair_of(slow)), self.rotary_dims - 1)
            ramp = ((idx - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            inv = inv / factor * ramp + inv * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.inv_freq = inv.to(torch.float32).to(device)

    def rotation(self, ctx):
        key = ("rope", id(self))
        hit = ctx.memo.get(key)
        if hit is None:
            half = self.rotary_dims // 2
            cos = ctx.buf(f"rope_cos_{id(self)}", (ctx.n_rows, half), torch.float32)
            sin = ctx.buf(f"rope_sin_{id(self)}", (ctx.n_rows, half), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, cos, sin)
            hit = (cos, sin)
            ctx.memo[key] = hit
        return hit


register_position("rope", Rope)
