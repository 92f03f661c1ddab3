"""Small Pimodra configurations and weights for the tests.

The configurations differ from one another in every size and option: norms in one to five groups, models with a looped
stretch at the start, in the middle, over everything, or without one, two to four passes, as many key/value heads as
heads, fewer, or one, key and value sizes that differ either way and fill a stored head or not, windows of one token
to more than a page and layers without a window, rotations of a whole head, of a part, without a stretch of the slow
pairs and without a rotation at all, score scales that are not the key size's inverse root, dense feed-forwards,
mixtures with and without groups, with one kept group and several, with one choice and several, layers without a
feed-forward.
"""
from __future__ import annotations

import json
import os

import torch


def rot(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims, "scaling": None}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attention(heads, kv_heads, dim, vdim, scale, window=None, rotation=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rotation is not None:
        m["rot"] = rotation
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def layer(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, groups=1, eps=1e-5, loop=None):
    c = {"architecture": "Pimodra", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# a looped stretch in the middle, three passes; values wider than keys; part of a head rotated, slow pairs stretched; a
# layer that sees everything; a mixture without groups taking half of its experts; one key/value head for four heads and no
# rotation; a layer without a feed-forward; a window of two tokens
PM_A = config(64, 300, [layer(attention(4, 2, 16, 24, 0.9, window=7, rotation=rot(8, 100.0, (2.0, 16, 4.0, 1.0))), dense(96)),
                        layer(attention(3, 3, 8, 8, 1.2, rotation=rot(8, 50.0)), moe(6, 3, 40)),
                        layer(attention(4, 1, 24, 10, 0.7, window=20)),
                        layer(attention(2, 2, 12, 6, 1.0, window=2, rotation=rot(12, 1000.0, (8.0, 64, 8.0, 2.0))), dense(50))],
              groups=2, eps=1e-6, loop=(1, 3, 3))

# no loop, norms in one group (the plain RMS norm); six heads over two; two kept groups of four; one choice of five; a
# window of one token (a layer that sees only itself)
PM_B = config(96, 257, [layer(attention(6, 2, 16, 16, 0.8, window=33, rotation=rot(16, 10000.0, (3.0, 40, 6.0, 1.5))), moe(8, 3, 24, groups=(4, 2))),
                        layer(attention(2, 1, 40, 20, 0.4, rotation=rot(20, 300.0)), dense(160)),
                        layer(attention(3, 3, 8, 12, 1.5, window=1), moe(5, 1, 64)),
                        layer(attention(4, 4, 24, 8, 0.6, window=5, rotation=rot(24, 500.0)), dense(64))], groups=1)

# everything looped, four passes; rows that are no multiple of 16 bytes (width 100); five heads, five groups of a row; a
# mixture of twelve in three groups of which one is kept; odd sizes everywhere
PM_C = config(100, 333, [layer(attention(5, 5, 10, 5, 1.1, window=9, rotation=rot(6, 20.0, (1.5, 8, 2.0, 0.5))), moe(12, 4, 30, groups=(3, 1))),
                         layer(attention(6, 3, 12, 14, 0.9, rotation=rot(12, 64.0)), dense(150))], groups=5, eps=1e-4, loop=(0, 2, 4))

# the smallest of everything, rows of 60 bytes in bfloat16: one head, a loop over the last layer only, two passes
PM_D = config(30, 101, [layer(attention(1, 1, 6, 5, 1.4, rotation=rot(2, 10.0)), dense(34)),
                        layer(attention(2, 1, 10, 6, 1.0, window=3, rotation=rot(10, 100.0, (2.0, 8, 1.0, 1.0))), moe(4, 2, 18, groups=(2, 2))),
                        layer(attention(2, 2, 4, 4, 2.0))], groups=3, loop=(2, 3, 2))

# sizes at which the tensor-core kernels run: rows of 512, heads of 64 and 128, pages of 64; windows below and above a page
PM_E = config(512, 3000, [layer(attention(8, 2, 64, 64, 0.4, window=100, rotation=rot(64, 10000.0, (4.0, 256, 16.0, 1.0))), dense(1024)),
                          layer(attention(4, 4, 128, 64, 0.3, rotation=rot(64, 5000.0)), moe(16, 4, 128, groups=(4, 2))),
                          layer(attention(8, 4, 32, 64, 0.6, window=40, rotation=rot(32, 1000.0, (2.0, 64, 8.0, 2.0))), moe(16, 2, 256)),
                          layer(attention(6, 2, 64, 32, 0.35, rotation=rot(32, 10000.0)), dense(768))], groups=8, loop=(1, 3, 2))

CASES = {"A": (PM_A, [5, 17, 23, 40, 11, 30], 4), "B": (PM_B, [1, 31, 40, 70, 9, 50], 8), "C": (PM_C, [3, 50, 64, 29, 77, 2], 16),
         "D": (PM_D, [4, 19, 1, 33, 8, 12], 4)}


def draw_tensors(cfg_dict: dict, seed: int) -> dict:
    """Random weights by tensor name (bfloat16), drawn here with torch's generator.  Norm weights lie around one, the
    activation's four numbers and the rows added before a pass are of order one so that each of them shows, router
    matrices are wide so that few choices are close calls, the heads' mixing matrix has entries of either sign and a
    strong diagonal.  Queries and keys are unit vectors by the design, so how sharp the attention is lies with the
    configuration's `scale` alone."""
    from kungfu_b200.api import load_config
    from kungfu_b200 import registry
    cfg = load_config(json.loads(json.dumps(cfg_dict)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in registry.find(cfg.architecture).tensor_specs(cfg):
        name = spec.name
        x = torch.randn(tuple(spec.shape), generator=g)
        if name.endswith(("norm1", "norm2", "norm1b", "norm2b", "final.norm")):
            x = 1.0 + 0.2 * x
        elif name.endswith("mix.talk"):
            x = torch.eye(spec.shape[0]) + 0.4 * x
        elif name.endswith("mlp.act"):
            x = torch.tensor([0.8, -0.5, 0.4, 0.1]) + 0.1 * x
        elif name == "loop.step":
            x = 0.5 * x
        elif name.endswith("router"):
            x = 4.0 * x / (spec.shape[-1] ** 0.5)
        elif name == "embed":
            x = 0.5 * x
        else:
            x = x / (spec.shape[-1] ** 0.5)                  # projections keep the spread of their input
        out[name] = x.to(torch.bfloat16)
    return out


def write_model(folder: str, cfg_dict: dict, seed: int) -> str:
    from kungfu_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), draw_tensors(cfg_dict, seed))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg_dict, f)
    return folder
