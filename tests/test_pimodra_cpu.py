"""Pimodra without a GPU: configuration and weights, the plain implementation's own mechanisms on hand-made inputs, and
the engine's host logic (pages, looped layer runs with a cache each, portions, mixed batches) with the kernels replaced
by the CPU stand-in, against the plain implementation."""
import json
import math

import pytest
import torch

import helpers
import pimodra_cases as pm
import plain_pimodra as pp
from kungfu_b200 import api, registry
from kungfu_b200.config.base import ConfigError
from kungfu_b200.weights.store import WeightError, WeightStore


def _runner(folder, page, max_tokens, max_requests=4):
    cfg, model = api.load_model(folder, dtype="float32", device="cpu")
    return api.make_runner(cfg, model, dtype="float32", device="cpu", page_size=page, max_tokens=max_tokens,
                           max_requests=max_requests, max_context=512)


def _rel(got, ref):
    assert got
    scale = max(float(r.abs().max()) for r in ref.values())
    return max(float((row - ref[rid][pos].float()).abs().max()) for (rid, pos), row in got.items()) / scale


def test_config_reads_every_size_and_round_trips():
    cfg = api.load_config(json.loads(json.dumps(pm.PM_A)))
    assert cfg.architecture == "Pimodra" and cfg.width == 64 and cfg.vocab == 300 and len(cfg.layers) == 4
    assert (cfg.norm_eps, cfg.norm_groups) == (1e-6, 2) and (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 3, 3)
    a = cfg.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window) == (4, 2, 16, 24, 0.9, 7)
    assert (a.rot.base, a.rot.dims, a.rot.scaling) == (100.0, 8, (2.0, 16.0, 4.0, 1.0))
    assert cfg.layers[1].mixer.window is None and cfg.layers[1].mixer.rot.scaling is None and cfg.layers[2].mixer.rot is None
    f = cfg.layers[1].mlp
    assert (f.kind, f.experts, f.top, f.groups, f.keep, f.ff) == ("moe", 6, 3, 1, 1, 40)
    assert cfg.layers[2].mlp is None and cfg.layers[0].mlp.ff == 96
    g = api.load_config(json.loads(json.dumps(pm.PM_B))).layers[0].mlp
    assert (g.groups, g.keep) == (4, 2)
    assert api.load_config(cfg.to_dict()) == cfg
    assert api.load_config(json.loads(json.dumps(cfg.to_dict()))) == cfg
    # one layer run per pass of the looped stretch, each with pages of its own
    assert [(s["layer"], s["pass"]) for s in cfg.state_summary()] == \
        [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None)]
    assert api.load_config(json.loads(json.dumps(pm.PM_B))).loop is None


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(groups={"count": 4, "keep": 1}), "groups"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["loop"].update(stop=9), "loop"),
])
def test_config_errors_name_the_key(change, word):
    raw = json.loads(json.dumps(pm.PM_A))
    change(raw)
    with pytest.raises(ConfigError) as e:
        api.load_config(raw)
    assert word in str(e.value)


def test_weights_bind_by_name_and_faults_are_listed_together():
    cfg = api.load_config(json.loads(json.dumps(pm.PM_A)))
    arch = registry.find("Pimodra")
    t = pm.draw_tensors(pm.PM_A, 1)
    assert t["loop.step"].shape == (3, 64) and t["l0.mix.talk"].shape == (4, 4) and t["l0.mix.g"].shape == (4 * 24, 64)
    assert t["l2.mix.k"].shape == (24, 64) and t["l0.mlp.act"].shape == (4,) and "l2.norm2" not in t and "l1.mlp.e5.down" in t
    model = arch.build(cfg, WeightStore.from_tensors(t, device="cpu", compute_dtype=torch.float32))
    assert len(model.schedule) == 8 and len({c.cache for c in model.schedule}) == 8
    assert [c.layer for c in model.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c.shift is not None for c in model.schedule] == [False, True, False, True, False, True, False, False]
    assert model.head.weight.data_ptr() == model.embedding.table.data_ptr()
    m = model.layers[0].mixer
    assert (m.key_dim, m.value_dim, m.window, m.position.rotary_dims) == (16, 24, 7, 8) and model.layers[2].mixer.position is None
    assert model.layers[0].mixer.position is not model.layers[1].mixer.position
    bad = dict(t)
    del bad["l1.mix.talk"]
    bad["l0.mix.g"] = torch.zeros(5, 64, dtype=torch.bfloat16)
    bad["extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as e:
        arch.build(cfg, WeightStore.from_tensors(bad, device="cpu", compute_dtype=torch.float32))
    assert "l1.mix.talk" in e.value.missing or any(n == "l0.mix.g" for n, _, _ in e.value.wrong_shape)


# ---- the plain implementation's mechanisms on inputs whose answers are known -------------------------------------------------

def test_plain_group_norm_by_hand():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0, 1.0, 1.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 1.0, 3.0, 1.0])
    y = pp.group_norm(x, w, 0.0, 3)
    r = math.sqrt(12.5)
    assert torch.allclose(y[0, :2], torch.tensor([3.0 / r, 8.0 / r], dtype=torch.float64))
    assert torch.allclose(y[0, 4:], torch.tensor([3.0, 1.0], dtype=torch.float64))
    one = pp.group_norm(x, torch.ones(6), 0.0, 1)
    assert abs(float((one * one).mean()) - 1.0) < 1e-12 and not torch.allclose(one, pp.group_norm(x, torch.ones(6), 0.0, 2))
    assert float(pp.group_norm(torch.zeros(1, 6, dtype=torch.float64), w, 1e-5, 3).abs().max()) == 0.0   # eps inside the root


def test_plain_rotation_frequencies_by_hand():
    f, mag = pp.yarn_frequencies({"base": 100.0, "dims": 8, "scaling": None})
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=torch.float64))
    # stretched: pair(t) = 8 ln(16 / (2 pi t)) / (2 ln 100); fast 0.25 turns -> 2.02.. floor 2; slow 0.05 -> 3.4.. ceil 4
    f2, mag2 = pp.yarn_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "original": 16, "fast": 0.25, "slow": 0.05}})
    assert abs(mag2 - (0.1 * math.log(2.0) + 1.0)) < 1e-15
    ramp = torch.tensor([0.0, 0.0, 0.0, 0.5], dtype=torch.float64)                 # lo 2, hi 4
    assert torch.allclose(f2, f / 2.0 * ramp + f * (1 - ramp))
    x = torch.zeros(3, 1, 10, dtype=torch.float64)
    x[:, 0, 0] = 1.0
    x[:, 0, 9] = 7.0
    y = pp.rotate(x, torch.tensor([0, 1, 5]), {"base": 100.0, "dims": 8, "scaling": None})
    assert torch.allclose(y[:, 0, 0], torch.cos(torch.tensor([0.0, 1.0, 5.0], dtype=torch.float64)))
    assert torch.allclose(y[:, 0, 4], torch.sin(torch.tensor([0.0, 1.0, 5.0], dtype=torch.float64)))      # the partner is i + r/2
    assert float((y[:, 0, 9] - 7.0).abs().max()) == 0.0 and float(y[:, 0, 8].abs().max()) == 0.0          # beyond r: as it was


def test_plain_router_by_hand():
    """Groups decide before experts do: the second largest score loses when its group's best is below the kept group's;
    the winners keep their softmax scores as weights."""
    z = torch.tensor([[2.0, 1.9, -5.0, 1.95, -5.0, -5.0]], dtype=torch.float64)
    ids, w = pp.route(z, 6, 2, 3, 1)
    s = torch.softmax(z[0], -1)
    assert sorted(ids[0].tolist()) == [0, 1]
    assert abs(float(w[0].sum()) - float(s[0] + s[1])) < 1e-15 and float(w[0].sum()) < 0.9
    ids, _ = pp.route(z, 6, 2, 3, 2)
    assert sorted(ids[0].tolist()) == [0, 3]
    ids, _ = pp.route(z, 6, 2, 1, 1)
    assert sorted(ids[0].tolist()) == [0, 3]


def test_plain_attention_sees_its_window_and_mixes_weights_after_the_softmax():
    g = torch.Generator().manual_seed(5)
    W, H, G, d, dv, T = 12, 4, 2, 6, 3, 9
    w = {"p.q": torch.randn(H * d, W, generator=g), "p.k": torch.randn(G * d, W, generator=g), "p.v": torch.randn(G * dv, W, generator=g),
         "p.g": torch.randn(H * dv, W, generator=g), "p.o": torch.eye(H * dv), "p.talk": torch.eye(H)}
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.7, "mask": {"size": 3}}
    base = pp.talking_attention(h, m, w, "p.", 1e-6)
    h2 = h.clone()
    h2[2] += 1.0                                                     # row 2 is seen by rows 2, 3, 4 and no later one
    moved = (pp.talking_attention(h2, m, w, "p.", 1e-6) - base).abs().amax(-1)
    assert float(moved[:2].max()) == 0.0 and float(moved[5:].max()) == 0.0 and float(moved[2:5].min()) > 1e-6
    # mixing with a permutation of heads hands head 1's weights to head 0: with one value head per query head and equal
    # value heads it would not show, so heads 0 and 1 share a value head here and the gate is neutralised
    w2 = dict(w)
    w2["p.talk"] = torch.eye(H)[[1, 0, 2, 3]]
    w2["p.g"] = w["p.g"] * 0
    w["p.g"] = w["p.g"] * 0
    a = pp.talking_attention(h, m, w, "p.", 1e-6).reshape(T, H, dv)
    b = pp.talking_attention(h, m, w2, "p.", 1e-6).reshape(T, H, dv)
    assert torch.allclose(a[:, 0], b[:, 1]) and torch.allclose(a[:, 1], b[:, 0]) and torch.allclose(a[:, 2:], b[:, 2:])
    # a mixing matrix of twice the identity doubles the result: weights are mixed after, not before, the softmax
    w2["p.talk"] = 2 * torch.eye(H)
    assert torch.allclose(pp.talking_attention(h, m, w2, "p.", 1e-6), 2 * a.reshape(T, H * dv))


def test_plain_activation_by_hand():
    z = torch.tensor([[1.0, -1.0, 2.0, 0.0]], dtype=torch.float64)
    y = pp.poly_norm(z, torch.tensor([1.0, 0.0, 0.0, 0.5]), 0.0)
    assert torch.allclose(y, z / math.sqrt(1.5) + 0.5)
    y = pp.poly_norm(z, torch.tensor([0.0, 2.0, 0.0, 0.0]), 0.0)
    assert torch.allclose(y, 2 * z * z / math.sqrt(18.0 / 4))
    y = pp.poly_norm(z, torch.tensor([0.0, 0.0, 1.0, 0.0]), 0.0)
    assert torch.allclose(y, z ** 3 / math.sqrt(66.0 / 4))


def test_plain_loop_adds_its_row_once_per_pass():
    cfg = json.loads(json.dumps(pm.PM_A))
    t = pm.draw_tensors(pm.PM_A, 2)
    toks = helpers.random_tokens(12, 300, 1)
    _, after = pp.forward(cfg, t, toks, keep_layers=True)
    assert after.shape == (8, 12, 64)
    t2 = dict(t)
    t2["loop.step"] = t["loop.step"].clone()
    t2["loop.step"][2] += 1.0                                        # the third pass starts at layer run 5
    _, after2 = pp.forward(cfg, t2, toks, keep_layers=True)
    assert float((after2[:5] - after[:5]).abs().max()) == 0.0 and float((after2[5] - after[5]).abs().max()) > 1e-3


# ---- the engine's host logic ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "chunks", "mixed"])
def test_host_logic_on_the_cpu_stand_in(name, mode, tmp_path, cpu_ops):
    cfg, lengths, page = pm.CASES[name]
    folder = pm.write_model(str(tmp_path / "m"), cfg, seed=3)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(lengths)}
    tensors = helpers.read_tensors(folder)
    ref = {rid: pp.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    steps = {"whole": helpers.trace_whole, "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=4)}[mode](reqs)
    runner = _runner(folder, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(lengths)
    assert _rel(got, ref) < 3e-4
    assert runner.cache.n_live == 0
    runner.cache.check()
