"""Nukelix hyperparameters, read from the model's own config.json.

A Nukelix file lists its layers one by one; nothing is implied by a layer's index and no size is fixed by the design.

  architecture            "Nukelix"
  width, vocab            residual width, vocabulary
  norm.eps                epsilon of every RMS norm
  logit_softcap           cap of the output logits (absent or 0: none)
  layers[i].type          attention | parallel | latent_attention
  layers[i].mixer         attention:        heads, kv_heads, dim (query/key head size), vdim (value head size), scale,
                                            mask {size, keep_first} (absent: every earlier token is seen),
                                            rot {base, dims, scaling {factor, low, high, original} | null}, v_mix
                          parallel:         left {heads, kv_heads, dim, vdim, scale, rot {base, dims}}, left_scale,
                                            right {heads, dim, vdim, gate_cap}, right_scale
                          latent_attention: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                                            rot {base, dims, scaling {factor, original, fast, slow} | null}
  layers[i].mlp           null | {kind: moe, expert {ff}, router {experts, top}, shared {ff} | null}
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

ATTENTION, PARALLEL, LATENT = "attention", "parallel", "latent_attention"


@dataclass(frozen=True)
class RotSpec:
    base: float
    dims: int
    scaling: tuple | None = None             # attention: (factor, low, high, original); latent: (factor, original, fast, slow)

    def wavelength_dict(self) -> dict | None:
        return dict(zip(("factor", "low", "high", "original"), self.scaling)) if self.scaling else None

    def ramp_dict(self) -> dict | None:
        return dict(zip(("factor", "original", "fast", "slow"), self.scaling)) if self.scaling else None


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotSpec | None = None
    window: int | None = None
    keep_first: int = 0
    v_mix: bool = False


@dataclass(frozen=True)
class MemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelSpec:
    left: AttentionSpec
    right: MemorySpec
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotSpec | None = None


@dataclass(frozen=True)
class MlpSpec:
    ff: int
    experts: int
    top: int
    shared_ff: int = 0                       # 0: no shared expert


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: object
    mlp: MlpSpec | None


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


def _rot(mk: KeyReader, default_dims: int, scaling_keys: tuple) -> RotSpec | None:
    rk = _sub(mk, "rot", required=False)
    if rk is None:
        return None
    sk = _sub(rk, "scaling", required=False)
    scaling = tuple(sk.float(key) for key in scaling_keys) if sk is not None else None
    rot = RotSpec(rk.float("base"), rk.int("dims", default_dims, min=0), scaling)
    return rot if rot.dims > 0 else None


def _attention(mk: KeyReader, windowed: bool) -> AttentionSpec:
    heads, dim = mk.int("heads", min=1), mk.int("dim", min=1)
    window, keep = None, 0
    mask = _sub(mk, "mask", required=False) if windowed else None
    if mask is not None:
        window = mask.int("size", None, min=1)
        keep = mask.int("keep_first", 0, min=0) if window is not None else 0
    return AttentionSpec(heads, mk.int("kv_heads", heads, min=1), dim, mk.int("vdim", dim, min=1), mk.float("scale"),
                         _rot(mk, dim, ("factor", "low", "high", "original")), window, keep,
                         mk.bool("v_mix", False) if windowed else False)


def _mixer(kind: str, mk: KeyReader):
    if kind == ATTENTION:
        return _attention(mk, True)
    if kind == PARALLEL:
        rk = _sub(mk, "right")
        right = MemorySpec(rk.int("heads", min=1), rk.int("dim", min=1), rk.int("vdim", min=1), rk.float("gate_cap"))
        return ParallelSpec(_attention(_sub(mk, "left"), False), right, mk.float("left_scale", 1.0), mk.float("right_scale", 1.0))
    rot_dim = mk.int("rot_dim", 0, min=0)
    return LatentSpec(mk.int("heads", min=1), mk.int("dim", min=1), rot_dim, mk.int("vdim", min=1), mk.int("kv_rank", min=1),
                      mk.int("q_rank", min=1), mk.float("scale"), _rot(mk, rot_dim, ("factor", "original", "fast", "slow")))


def _mlp(k: KeyReader | None) -> MlpSpec | None:
    if k is None:
        return None
    k.str("kind", "moe", choices=("moe",))
    r = _sub(k, "router")
    sh = _sub(k, "shared", required=False)
    return MlpSpec(_sub(k, "expert").int("ff", min=1), r.int("experts", min=1), r.int("top", min=1),
                   sh.int("ff", min=1) if sh is not None else 0)


@dataclass(frozen=True)
class NukelixConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    logit_softcap: float = 0.0
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
    def from_dict(cls, raw: dict, where: str = "config.json") -> "NukelixConfig":
        k = KeyReader(raw, where)
        arch = k.str("architecture")
        width, vocab = k.int("width", min=1), k.int("vocab", min=1)
        eps = _sub(k, "norm").float("eps")
        layers = []
        for i, e in enumerate(k.list("layers")):
            ek = KeyReader(e, f"{where}: layers[{i}]")
            kind = ek.str("type", choices=(ATTENTION, PARALLEL, LATENT))
            layers.append(LayerSpec(kind, _mixer(kind, _sub(ek, "mixer")), _mlp(_sub(ek, "mlp", required=False))))
        cfg = cls(arch, width, vocab, eps, k.float("logit_softcap", 0.0) or 0.0, tuple(layers))
        cfg.validate(where)
        return cfg

    def v_mix_layers(self) -> list:
        """The layers whose values are mixed, in order; the first of them gives, the others take."""
        return [i for i, l in enumerate(self.layers) if l.type == ATTENTION and l.mixer.v_mix]

    def validate(self, where: str = "config") -> None:
        if not self.layers:
            raise ConfigError(f"{where}: 'layers' is empty")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{where}: norm.eps must be positive, found {self.norm_eps}")

        def check_attention(m: AttentionSpec, at: str) -> None:
            if m.heads % m.kv_heads:
                raise ConfigError(f"{at}: heads {m.heads} is not a multiple of kv_heads {m.kv_heads}")
            if max(m.dim, m.vdim) > 256:
                raise ConfigError(f"{at}: head sizes above 256 are not supported, found {max(m.dim, m.vdim)}")
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                raise ConfigError(f"{at}: rot.dims {m.rot.dims} must be even and at most dim {m.dim}")

        for i, l in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            m = l.mixer
            if l.type == ATTENTION:
                check_attention(m, at)
            elif l.type == PARALLEL:
                check_attention(m.left, at + ": left")
                if m.right.dim > 256:
                    raise ConfigError(f"{at}: right: key size {m.right.dim} is above 256")
                if not m.right.gate_cap > 0:
                    raise ConfigError(f"{at}: right: gate_cap must be positive, found {m.right.gate_cap}")
            else:
                if m.kv_rank + m.rot_dim > 512:
                    raise ConfigError(f"{at}: kv_rank + rot_dim above 512 is not supported, found {m.kv_rank + m.rot_dim}")
                if m.rot_dim % 2 or (m.rot is not None and m.rot.dims != m.rot_dim):
                    raise ConfigError(f"{at}: rot_dim {m.rot_dim} must be even and equal to rot.dims")
                if (m.rot is None) != (m.rot_dim == 0):
                    raise ConfigError(f"{at}: rot_dim {m.rot_dim} and 'rot' do not agree")
            f = l.mlp
            if f is not None:
                if f.top > f.experts:
                    raise ConfigError(f"{at}: mlp: top {f.top} of {f.experts} experts")
                if f.experts > 1024:
                    raise ConfigError(f"{at}: mlp: more than 1024 experts are not supported")
        mixed = self.v_mix_layers()
        if mixed:
            first = self.layers[mixed[0]].mixer
            for i in mixed[1:]:
                m = self.layers[i].mixer
                if (m.kv_heads, m.vdim) != (first.kv_heads, first.vdim):
                    raise ConfigError(f"{where}: layers[{i}]: values of {m.kv_heads} x {m.vdim} cannot be mixed with "
                                      f"layer {mixed[0]}'s {first.kv_heads} x {first.vdim}")

    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to this configuration."""

        def rot(r: RotSpec | None, d):
            return None if r is None else {"base": r.base, "dims": r.dims, "scaling": d(r)}

        def attention(m: AttentionSpec, windowed: bool) -> dict:
            out = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                   "rot": rot(m.rot, RotSpec.wavelength_dict)}
            if windowed:
                out["v_mix"] = m.v_mix
                if m.window is not None:
                    out["mask"] = {"size": m.window, "keep_first": m.keep_first}
            return out

        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == ATTENTION:
                mixer = attention(m, True)
            elif l.type == PARALLEL:
                mixer = {"left": attention(m.left, False), "left_scale": m.left_scale, "right_scale": m.right_scale,
                         "right": {"heads": m.right.heads, "dim": m.right.dim, "vdim": m.right.vdim, "gate_cap": m.right.gate_cap}}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                         "q_rank": m.q_rank, "scale": m.scale, "rot": rot(m.rot, RotSpec.ramp_dict)}
            f = l.mlp
            mlp = None if f is None else {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top},
                                          "shared": {"ff": f.shared_ff} if f.shared_ff else None}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
                "logit_softcap": self.logit_softcap, "layers": layers}

    def replace(self, **kw) -> "NukelixConfig":
        cfg = dataclasses.replace(self, **kw)
        cfg.validate()
        return cfg

    def state_summary(self, element_size: int = 2) -> list:
        """Per layer, what it keeps per request: bytes per token of its pages, the window that bounds them, fixed bytes."""
        from ..ops import attention_head_size, mlstm_norm_width
        from ..parts.latent import latent_head_size
        out = []
        for i, l in enumerate(self.layers):
            m = l.mixer
            if l.type == LATENT:
                out.append({"layer": i, "kind": "latent_pages", "window": None, "fixed_bytes": 0,
                            "bytes_per_token": 2 * latent_head_size(m.kv_rank + m.rot_dim) * element_size})
                continue
            a = m if l.type == ATTENTION else m.left
            fixed = 0
            if l.type == PARALLEL:
                fixed = 4 * m.right.heads * (m.right.dim * m.right.vdim + mlstm_norm_width(m.right.dim, m.right.vdim))
            out.append({"layer": i, "kind": "kv_pages" if not fixed else "kv_pages+memory", "window": a.window,
                        "fixed_bytes": fixed,
                        "bytes_per_token": 2 * a.kv_heads * attention_head_size(max(a.dim, a.vdim)) * element_size})
        return out
