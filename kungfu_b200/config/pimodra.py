"""Pimodra hyperparameters, read from the model's own config.json.

A Pimodra file lists its layers one by one; nothing is implied by a layer's index and no size is fixed by the design.

  architecture            "Pimodra"
  width, vocab            residual width, vocabulary
  norm.eps, norm.groups   epsilon of every RMS norm; into how many equal parts a norm cuts its row (default 1)
  loop                    null | {start, stop, times}: layers start .. stop-1 run `times` times in a row with the same
                          weights and a cache of their own per pass; tensor `loop.step` [times, width] holds the row that
                          is added to the residual before each pass
  layers[i].type          attention
  layers[i].mixer         heads, kv_heads, dim (query/key head size), vdim (value head size), scale,
                          mask {size} (sliding window; absent: every earlier token is seen),
                          rot {base, dims, scaling {factor, original, fast, slow} | null} (absent: no rotation)
  layers[i].mlp           null | {kind: dense, ff} | {kind: moe, expert {ff}, router {experts, top, groups {count, keep}}}
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

ATTENTION = "attention"


@dataclass(frozen=True)
class RotSpec:
    base: float
    dims: int
    scaling: tuple | None = None             # (factor, original, fast, slow)

    def yarn_dict(self) -> dict | None:
        if self.scaling is None:
            return None
        return dict(zip(("factor", "original", "fast", "slow"), self.scaling))


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
    rot: RotSpec | None


@dataclass(frozen=True)
class MlpSpec:
    kind: str                                # dense | moe
    ff: int = 0                              # dense: inner size; moe: inner size of one expert
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: AttentionSpec
    mlp: MlpSpec | None


@dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


def _sub(k: KeyReader, key: str, required: bool = True) -> KeyReader | None:
    raw = k.raw.get(key)
    k.read.add(key)
    if raw is None:
        if required:
            raise ConfigError(f"{k.where}: required key '{key}' is missing")
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"{k.where}: key '{key}' must be an object, found {raw!r}")
    return KeyReader(raw, f"{k.where}: {key}")


def _mlp(k: KeyReader | None) -> MlpSpec | None:
    if k is None:
        return None
    kind = k.str("kind", "dense", choices=("dense", "moe"))
    if kind == "dense":
        return MlpSpec("dense", ff=k.int("ff", min=1))
    r = _sub(k, "router")
    g = _sub(r, "groups", required=False)
    return MlpSpec("moe", ff=_sub(k, "expert").int("ff", min=1), experts=r.int("experts", min=1), top=r.int("top", min=1),
                   groups=g.int("count", 1, min=1) if g is not None else 1, keep=g.int("keep", 1, min=1) if g is not None else 1)


def _attention(mk: KeyReader) -> AttentionSpec:
    heads = mk.int("heads", min=1)
    dim = mk.int("dim", min=1)
    mask = _sub(mk, "mask", required=False)
    window = mask.int("size", None, min=1) if mask is not None else None
    rk = _sub(mk, "rot", required=False)
    rot = None
    if rk is not None:
        sk = _sub(rk, "scaling", required=False)
        scaling = None
        if sk is not None:
            scaling = (sk.float("factor"), sk.float("original"), sk.float("fast"), sk.float("slow"))
        rot = RotSpec(rk.float("base"), rk.int("dims", dim, min=0), scaling)
        if rot.dims == 0:
            rot = None
    return AttentionSpec(heads, mk.int("kv_heads", heads, min=1), dim, mk.int("vdim", dim, min=1), mk.float("scale"), window, rot)


@dataclass(frozen=True)
class PimodraConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    norm_groups: int = 1
    loop: LoopSpec | None = None
    layers: tuple = field(default_factory=tuple)         # LayerSpec per layer

    # what the engine and the command line ask of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "PimodraConfig":
        k = KeyReader(raw, where)
        arch = k.str("architecture")
        width, vocab = k.int("width", min=1), k.int("vocab", min=1)
        nk = _sub(k, "norm")
        eps, groups = nk.float("eps"), nk.int("groups", 1, min=1)
        lk = _sub(k, "loop", required=False)
        loop = LoopSpec(lk.int("start", min=0), lk.int("stop", min=0), lk.int("times", min=1)) if lk is not None else None
        layers = []
        for i, e in enumerate(k.list("layers")):
            ek = KeyReader(e, f"{where}: layers[{i}]")
            kind = ek.str("type", choices=(ATTENTION,))
            layers.append(LayerSpec(kind, _attention(_sub(ek, "mixer")), _mlp(_sub(ek, "mlp", required=False))))
        cfg = cls(arch, width, vocab, eps, groups, loop, tuple(layers))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if not self.layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{where}: norm.eps must be positive, found {self.norm_eps}")
        if self.width % self.norm_groups:
            raise ConfigError(f"{where}: norm.groups {self.norm_groups} does not divide width {self.width}")
        if self.loop is not None and not (0 <= self.loop.start <= self.loop.stop <= len(self.layers)):
            raise ConfigError(f"{where}: loop {self.loop.start}..{self.loop.stop} does not lie within {len(self.layers)} layers")
        for i, l in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            m = l.mixer
            if m.heads % m.kv_heads:
                raise ConfigError(f"{at}: heads {m.heads} is not a multiple of kv_heads {m.kv_heads}")
            if max(m.dim, m.vdim) > 256:
                raise ConfigError(f"{at}: head sizes above 256 are not supported, found {max(m.dim, m.vdim)}")
            if m.heads > 128:
                raise ConfigError(f"{at}: more than 128 heads are not supported")
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                raise ConfigError(f"{at}: rot.dims {m.rot.dims} must be even and at most dim {m.dim}")
            f = l.mlp
            if f is not None and f.kind == "moe":
                if f.top > f.experts or f.experts % f.groups or not (1 <= f.keep <= f.groups):
                    raise ConfigError(f"{at}: mlp: {f.experts} experts, top {f.top}, groups {f.groups}, keep {f.keep} do not fit")
                if f.groups > 1 and f.keep * (f.experts // f.groups) < f.top:
                    raise ConfigError(f"{at}: mlp: {f.keep} groups of {f.experts // f.groups} experts cannot give {f.top} choices")
                if f.experts > 1024:
                    raise ConfigError(f"{at}: mlp: more than 1024 experts are not supported")

    def layer_runs(self) -> list:
        """[(layer, pass number or None)] in running order: the looped stretch `times` times, the rest once."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop <= self.loop.start:
            return [(i, None) for i in range(n)]
        lp = self.loop
        runs = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to this configuration."""
        layers = []
        for l in self.layers:
            m = l.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.window is not None:
                mixer["mask"] = {"size": m.window}
            if m.rot is not None:
                mixer["rot"] = {"base": m.rot.base, "dims": m.rot.dims, "scaling": m.rot.yarn_dict()}
            f = l.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "groups": {"count": f.groups, "keep": f.keep}}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    def replace(self, **kw) -> "PimodraConfig":
        cfg = dataclasses.replace(self, **kw)
        cfg.validate()
        return cfg

    def state_summary(self, element_size: int = 2) -> list:
        """Per layer run, what it keeps per request: bytes per token of its pages and the window that bounds them."""
        from ..ops import attention_head_size
        out = []
        for i, t in self.layer_runs():
            m = self.layers[i].mixer
            stored = m.kv_heads
            out.append({"layer": i, "pass": t, "kind": "kv_pages", "window": m.window, "fixed_bytes": 0,
                        "bytes_per_token": 2 * stored * attention_head_size(max(m.dim, m.vdim)) * element_size})
        return out
