"""Small Nukelix configurations and weights for the tests.

The configurations differ from one another in every size and option: each kind of layer first, last, twice in a row or
absent; as many key/value heads as heads, fewer, or one; key and value sizes that differ either way; windows of two
tokens to more than a page, with no kept first tokens, a few, or more than the window; layers of the windowed kind
without a mask; rotations of a whole head, of a part, with and without rescaling (all three regimes of the wavelength
rule reached, ramps that start at pair 0 and later); value mixing over two and three layers and none; memories of one to
four heads with key sizes 4 to 64; latents that fill their stored head or not, query latents smaller and larger than the
key latent; mixtures with one choice, several and all experts, with and without a shared expert; layers without a
feed-forward; widths that are no multiple of 16 bytes.
"""
from __future__ import annotations

import json
import os

import torch


def rot(dims, base=10000.0, scaling=None, keys=("factor", "low", "high", "original")):
    return {"base": base, "dims": dims, "scaling": dict(zip(keys, scaling)) if scaling else None}


def ramp_rot(dims, base=10000.0, scaling=None):
    return rot(dims, base, scaling, ("factor", "original", "fast", "slow"))


def attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=0, rotation=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rotation is not None:
        m["rot"] = rotation
    return m


def left(heads, kv_heads, dim, vdim, scale, rotation=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rotation is not None:
        m["rot"] = rotation
    return m


def parallel(left_mixer, right_heads, right_dim, right_vdim, cap, left_scale=1.0, right_scale=1.0):
    return {"left": left_mixer, "left_scale": left_scale, "right_scale": right_scale,
            "right": {"heads": right_heads, "dim": right_dim, "vdim": right_vdim, "gate_cap": cap}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if rot_dim:
        m["rot"] = ramp_rot(rot_dim, base, scaling)
    return m


def moe(experts, top, ff, shared=0):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": {"ff": shared} if shared else None}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, eps=1e-5, softcap=20.0):
    return {"architecture": "Nukelix", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_softcap": softcap,
            "layers": layers}


# every kind of layer; values wider than keys; three kept tokens behind a window of seven; values mixed over two layers;
# a latent layer without a feed-forward; a mixture without a shared expert
NK_A = config(64, 300, [
    layer("attention", attention(4, 2, 16, 24, 0.3, window=7, keep_first=3, rotation=rot(8, 100.0, (3.0, 1.0, 4.0, 64)), v_mix=True),
          moe(6, 2, 40, shared=24)),
    layer("parallel", parallel(left(3, 3, 8, 8, 0.5, rot(8, 50.0)), 2, 8, 12, 8.0, 0.7, 1.1), moe(4, 4, 16)),
    layer("latent_attention", latent(3, 8, 4, 6, 20, 12, 0.4, 1000.0, (2.0, 16, 4.0, 1.0))),
    layer("attention", attention(2, 2, 12, 24, 0.35, window=20, keep_first=5, rotation=rot(12, 1000.0), v_mix=True),
          moe(5, 1, 30))], eps=1e-6)

# the memory first; a windowed layer that keeps nothing; a latent whose queries' latent is the larger one; a layer of
# the windowed kind without a mask (every earlier token and the sink); no mixing anywhere; no cap on the logits
NK_B = config(96, 257, [
    layer("parallel", parallel(left(6, 2, 16, 8, 0.25, rot(16, 10000.0)), 4, 4, 16, 15.0, 1.0, 0.5), moe(8, 3, 24, shared=48)),
    layer("attention", attention(6, 3, 8, 16, 0.5, window=33, keep_first=0, rotation=rot(4, 300.0, (8.0, 1.0, 2.0, 32)))),
    layer("latent_attention", latent(2, 24, 8, 20, 16, 40, 0.2, 500.0), moe(3, 2, 64, shared=16)),
    layer("attention", attention(4, 4, 24, 8, 0.2), moe(7, 2, 20, shared=20))], eps=1e-5, softcap=0.0)

# rows that are no multiple of 16 bytes (width 100); five heads; odd sizes; more kept tokens than the window is long; values
# mixed over three layers; two memories in a row
NK_C = config(100, 333, [
    layer("attention", attention(5, 5, 10, 6, 0.3, window=4, keep_first=6, rotation=rot(6, 20.0, (2.0, 0.5, 3.0, 40)), v_mix=True),
          moe(12, 5, 30, shared=10)),
    layer("attention", attention(5, 5, 6, 6, 0.5, window=9, keep_first=1, v_mix=True)),
    layer("parallel", parallel(left(6, 3, 12, 14, 0.3, rot(6, 64.0)), 3, 10, 6, 5.0, 1.3, 0.4), moe(4, 1, 50)),
    layer("parallel", parallel(left(2, 1, 20, 10, 0.25), 1, 16, 20, 30.0, 0.5, 1.5)),
    layer("attention", attention(10, 5, 4, 6, 0.6, window=30, keep_first=2, rotation=rot(4, 9.0), v_mix=True), moe(2, 2, 44, shared=44))],
    eps=1e-4, softcap=8.0)

# the smallest of everything, rows of 60 bytes in bfloat16: one head, a window of two tokens
NK_D = config(30, 101, [
    layer("latent_attention", latent(1, 6, 2, 5, 7, 3, 0.7, 10.0, (4.0, 8, 1.0, 1.0)), moe(2, 1, 18)),
    layer("attention", attention(1, 1, 6, 5, 0.6, window=2, keep_first=1, rotation=rot(2, 10.0)), moe(3, 2, 12, shared=7)),
    layer("parallel", parallel(left(2, 1, 10, 6, 0.4, rot(10, 100.0)), 1, 4, 4, 3.0, 0.9, 0.9))], softcap=50.0)

# sizes at which the tensor-core kernels run: rows of 512, heads of 64 and 128, pages of 64; windows below and above a page
NK_E = config(512, 3000, [
    layer("attention", attention(8, 2, 64, 64, 0.1, window=100, keep_first=10, rotation=rot(32, 10000.0, (4.0, 1.0, 4.0, 256)), v_mix=True),
          moe(16, 4, 128, shared=256)),
    layer("parallel", parallel(left(4, 4, 128, 64, 0.07, rot(64, 5000.0)), 4, 64, 64, 10.0, 0.8, 1.2), moe(8, 2, 256)),
    layer("latent_attention", latent(8, 32, 32, 64, 96, 64, 0.12, 1000.0, (2.0, 64, 8.0, 2.0)), moe(16, 1, 64, shared=128)),
    layer("attention", attention(4, 2, 32, 64, 0.15, window=40, keep_first=70, rotation=rot(32, 1000.0), v_mix=True), moe(4, 3, 192)),
    layer("parallel", parallel(left(8, 2, 64, 32, 0.1, rot(32, 10000.0)), 2, 32, 128, 11.0, 1.1, 0.6))], eps=1e-6, softcap=25.0)

CASES = {"A": (NK_A, [5, 17, 23, 40, 11, 30], 4), "B": (NK_B, [1, 31, 40, 70, 9, 50], 8), "C": (NK_C, [3, 50, 64, 29, 77, 2], 16),
         "D": (NK_D, [4, 19, 1, 33, 8, 12], 4)}


def draw_tensors(cfg_dict: dict, seed: int, sharp: float = 1.0) -> dict:
    """Random weights by tensor name (bfloat16), drawn here with torch's generator.  Norm weights lie around one; the
    weights of the norms over q and k around `sharp`, which spreads the scores; biases are of the order of the
    projections; mixing numbers lie between 0.2 and 0.6; router matrices are wide so that few choices are close calls;
    forget-gate biases are large so that hundreds of tokens weigh in a memory."""
    from kungfu_b200.api import load_config
    from kungfu_b200 import registry
    cfg = load_config(json.loads(json.dumps(cfg_dict)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in registry.find(cfg.architecture).tensor_specs(cfg):
        name = spec.name
        x = torch.randn(tuple(spec.shape), generator=g)
        if name.endswith(("q.norm", "k.norm")):
            x = sharp * (1.0 + 0.2 * x)
        elif name.endswith("norm") or name.endswith(("norm1", "norm2")):
            x = 1.0 + 0.2 * x
        elif name.endswith("vmix"):
            x = 0.4 + 0.1 * x.clamp(-2, 2)
        elif name.endswith("f.b"):
            x = 4.0 + x
        elif name.endswith(".b"):
            x = 0.3 * x
        elif name.endswith("router"):
            x = 4.0 * x / (spec.shape[-1] ** 0.5)
        elif name == "embed":
            x = 0.5 * x
        else:
            x = x / (spec.shape[-1] ** 0.5)                  # projections keep the spread of their input
        out[name] = x.to(torch.bfloat16)
    return out


def write_tensors(folder: str, cfg_dict: dict, tensors: dict) -> str:
    from kungfu_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg_dict, f)
    return folder


def write_model(folder: str, cfg_dict: dict, seed: int, sharp: float = 1.0) -> str:
    return write_tensors(folder, cfg_dict, draw_tensors(cfg_dict, seed, sharp))
