"""Nukelix without a GPU: configuration and weights, the plain implementation's own mechanisms on hand-made inputs, and
the engine's host logic (pages with kept first tokens, state slots of the memories, portions, mixed batches) with the
kernels replaced by the CPU stand-in, against the plain implementation."""
import json
import math

import pytest
import torch

import helpers
import nukelix_cases as nk
import plain_nukelix as pn
from kungfu_b200 import api, registry
from kungfu_b200.config.base import ConfigError
from kungfu_b200.weights.store import WeightError, WeightStore

D64 = torch.float64


def _runner(folder, page, max_tokens, max_requests=4):
    cfg, model = api.load_model(folder, dtype="float32", device="cpu")
    return api.make_runner(cfg, model, dtype="float32", device="cpu", page_size=page, max_tokens=max_tokens,
                           max_requests=max_requests, max_context=512)


def _rel(got, ref):
    assert got
    scale = max(float(r.abs().max()) for r in ref.values())
    return max(float((row - ref[rid][pos].float()).abs().max()) for (rid, pos), row in got.items()) / scale


def test_config_reads_every_size_and_round_trips():
    cfg = api.load_config(json.loads(json.dumps(nk.NK_A)))
    assert cfg.architecture == "Nukelix" and cfg.width == 64 and cfg.vocab == 300 and len(cfg.layers) == 4
    assert cfg.norm_eps == 1e-6 and cfg.logit_softcap == 20.0
    a = cfg.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first, a.v_mix) == (4, 2, 16, 24, 0.3, 7, 3, True)
    assert (a.rot.base, a.rot.dims, a.rot.scaling) == (100.0, 8, (3.0, 1.0, 4.0, 64.0))
    p = cfg.layers[1].mixer
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.window, p.left_scale, p.right_scale) == (3, 3, 8, None, 0.7, 1.1)
    assert (p.right.heads, p.right.dim, p.right.vdim, p.right.gate_cap) == (2, 8, 12, 8.0)
    l = cfg.layers[2].mixer
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.q_rank, l.rot.scaling) == (3, 8, 4, 6, 20, 12, (2.0, 16.0, 4.0, 1.0))
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp.shared_ff == 0 and cfg.layers[0].mlp.shared_ff == 24
    f = cfg.layers[1].mlp
    assert (f.experts, f.top, f.ff) == (4, 4, 16)
    assert cfg.v_mix_layers() == [0, 3]
    assert api.load_config(cfg.to_dict()) == cfg
    assert api.load_config(json.loads(json.dumps(cfg.to_dict()))) == cfg
    b = api.load_config(json.loads(json.dumps(nk.NK_B)))
    assert b.layers[3].mixer.window is None and b.layers[3].mixer.rot is None and b.logit_softcap == 0.0 and b.v_mix_layers() == []
    kinds = [s["kind"] for s in cfg.state_summary()]
    assert kinds == ["kv_pages", "kv_pages+memory", "latent_pages", "kv_pages"]
    assert cfg.state_summary()[1]["fixed_bytes"] == 4 * 2 * (8 * 12 + 8 + 4)


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][2]["mixer"].update(rot_dim=6), "rot_dim"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=12), "mixed"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = json.loads(json.dumps(nk.NK_A))
    change(raw)
    with pytest.raises(ConfigError) as e:
        api.load_config(raw)
    assert word in str(e.value)


def test_weights_bind_by_name_and_faults_are_listed_together():
    cfg = api.load_config(json.loads(json.dumps(nk.NK_A)))
    arch = registry.find("Nukelix")
    t = nk.draw_tensors(nk.NK_A, 1)
    assert t["l0.mix.q.norm"].shape == (64,) and t["l0.mix.k.b"].shape == (32,) and t["l0.mix.vmix"].shape == ()
    assert t["l1.mix.right.norm"].shape == (24,) and t["l1.mix.right.f.b"].shape == (2,) and t["l1.mix.left.g"].shape == (3, 64)
    assert t["l2.mix.dkv"].shape == (24, 64) and t["l2.mix.uq"].shape == (36, 12) and "l2.norm2" not in t and "l3.mlp.shared.up" not in t
    model = arch.build(cfg, WeightStore.from_tensors(t, device="cpu", compute_dtype=torch.float32))
    assert model.head.weight.data_ptr() == model.embedding.table.data_ptr() and model.head.softcap == 20.0
    m0, m3 = model.layers[0].mixer, model.layers[3].mixer
    assert (m0.key_dim, m0.value_dim, m0.window, m0.keep_first, m0.sink, m0.v_mix) == (16, 24, 7, 3, True, "first")
    assert m3.v_mix == "mix" and m3.v_mix_weight.numel() == 1 and m0.position.interleaved and m0.position.scaling
    side = model.layers[1].mixer
    assert not side.left.sink and side.left.window is None and not side.left.position.interleaved
    assert (side.left_scale, side.right_scale, side.right.gate_cap) == (0.7, 1.1, 8.0)
    lat = model.layers[2].mixer
    assert lat.head_dim == 32 and lat.rot_dim == 4 and lat.position.magnitude == pytest.approx(0.1 * math.log(2.0) + 1.0)
    assert model.layers[0].ffn.weight_on == "input" and model.layers[0].ffn.shared is not None and model.layers[3].ffn.shared is None
    # what the cache manager is asked for: pages with kept first tokens; pages and two fixed states; pages of the latent
    needs = model.state_needs()
    assert (needs[0].window, needs[0].keep_first) == (7, 3) and len(needs[1].parts) == 2 and needs[2].n_kv_heads == 1
    bad = dict(t)
    del bad["l1.mix.right.i.b"]
    bad["l0.mix.g"] = torch.zeros(5, 64, dtype=torch.bfloat16)
    bad["extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as e:
        arch.build(cfg, WeightStore.from_tensors(bad, device="cpu", compute_dtype=torch.float32))
    assert "l1.mix.right.i.b" in e.value.missing or any(n == "l0.mix.g" for n, _, _ in e.value.wrong_shape)


# ---- the plain implementation's mechanisms on inputs whose answers are known -------------------------------------------------

def test_plain_frequencies_by_hand():
    r = {"base": 100.0, "dims": 8, "scaling": None}
    f = pn.plain_frequencies(r)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=D64))
    # by wavelength: 6.28 stays (below 64 / 4), 198.7 is divided (above 64 / 1), the two between are blended
    r["scaling"] = {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 64}
    g = pn.wavelength_scaled_frequencies(r)
    assert float(g[0]) == 1.0 and float(g[3]) == pytest.approx(float(f[3]) / 3.0)
    s1 = (64 * float(f[1]) / (2 * math.pi) - 1.0) / 3.0
    assert float(g[1]) == pytest.approx((1 - s1) * float(f[1]) / 3.0 + s1 * float(f[1])) and float(f[1]) / 3 < float(g[1]) < float(f[1])
    # by pair index: pair(t) = 8 ln(16 / (2 pi t)) / (2 ln 100); fast 0.25 turns -> 2.02.. floor 2; slow 0.05 -> 3.4.. ceil 4
    h, mag = pn.ramp_scaled_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "original": 16, "fast": 0.25, "slow": 0.05}})
    ramp = torch.tensor([0.0, 0.0, 0.0, 0.5], dtype=D64)
    assert mag == pytest.approx(0.1 * math.log(2.0) + 1.0) and torch.allclose(h, f / 2.0 * ramp + f * (1 - ramp))


def test_plain_rotation_pairs_by_hand():
    x = torch.zeros(3, 1, 10, dtype=D64)
    x[:, 0, 0] = 1.0
    x[:, 0, 9] = 7.0
    pos = torch.tensor([0, 1, 5])
    f = pn.plain_frequencies({"base": 100.0, "dims": 8})
    ang = torch.tensor([0.0, 1.0, 5.0], dtype=D64)
    y = pn.rotate(x, pos, f, 8, False)
    assert torch.allclose(y[:, 0, 0], torch.cos(ang)) and torch.allclose(y[:, 0, 4], torch.sin(ang))      # partner i + r/2
    z = pn.rotate(x, pos, f, 8, True, 1.5)
    assert torch.allclose(z[:, 0, 0], 1.5 * torch.cos(ang)) and torch.allclose(z[:, 0, 1], 1.5 * torch.sin(ang))   # partner 2i + 1
    assert float(z[:, 0, 4].abs().max()) == 0.0
    for out in (y, z):
        assert float((out[:, 0, 9] - 7.0).abs().max()) == 0.0 and float(out[:, 0, 8].abs().max()) == 0.0  # beyond r: as it was


def test_plain_mask_and_sink_by_hand():
    m = pn.visible(7, 3, 2)
    assert m[6].tolist() == [True, True, False, False, True, True, True]          # two kept, then the window of three
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert pn.visible(7, 3, 0)[6].tolist() == [False, False, False, False, True, True, True]
    assert pn.visible(4, None, 5)[3].tolist() == [True] * 4
    # one key of score ln 3 and the sink: weights 3 / (3 + 1); without the sink a lone key has weight one
    q = torch.tensor([[[math.log(3.0)]]], dtype=D64)
    k = torch.ones(1, 1, 1, dtype=D64)
    v = torch.tensor([[[2.0, -4.0]]], dtype=D64)
    assert torch.allclose(pn.attend(q, k, v, 1.0, pn.visible(1, None, 0), True)[0, 0], 0.75 * v[0, 0])
    assert torch.allclose(pn.attend(q, k, v, 1.0, pn.visible(1, None, 0), False)[0, 0], v[0, 0])
    # scores far below zero: the sink takes nearly everything
    assert float(pn.attend(-20 * q, k, v, 1.0, pn.visible(1, None, 0), True).abs().max()) < 1e-8


def test_plain_attention_norms_over_all_heads_and_mixes_values():
    g = torch.Generator().manual_seed(5)
    W, H, G, d, dv, T = 12, 4, 2, 6, 3, 9
    w = {"p.q": torch.randn(H * d, W, generator=g), "p.k": torch.randn(G * d, W, generator=g), "p.v": torch.randn(G * dv, W, generator=g),
         "p.q.b": torch.randn(H * d, generator=g), "p.k.b": torch.randn(G * d, generator=g), "p.v.b": torch.randn(G * dv, generator=g),
         "p.q.norm": torch.ones(H * d), "p.k.norm": torch.ones(G * d), "p.g": torch.zeros(H, W), "p.o": torch.eye(H * dv),
         "p.vmix": torch.tensor(0.25)}
    h = torch.randn(T, W, generator=g, dtype=D64)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.7, "mask": {"size": 3, "keep_first": 1}, "v_mix": True}
    q, k, v = pn.gqa_projections(h, w, "p.", m, 0.0)
    assert torch.allclose((q * q).mean((1, 2)), torch.ones(T, dtype=D64)) and not torch.allclose((q * q).mean(2), torch.ones(T, H, dtype=D64))
    pos = torch.arange(T)
    base, v0 = pn.windowed_attention(h, w, "p.", m, 0.0, pos, None)
    assert torch.allclose(v0, v)
    h2 = h.clone()
    h2[2] += 1.0                                             # row 2 is seen by rows 2, 3, 4; row 0 by every row
    moved = (pn.windowed_attention(h2, w, "p.", m, 0.0, pos, None)[0] - base).abs().amax(-1)
    assert float(moved[:2].max()) == 0.0 and float(moved[5:].max()) == 0.0 and float(moved[2:5].min()) > 1e-6
    h3 = h.clone()
    h3[0] += 1.0
    assert float((pn.windowed_attention(h3, w, "p.", m, 0.0, pos, None)[0] - base).abs().amax(-1).min()) > 1e-7
    first = torch.randn(T, G, dv, generator=g, dtype=D64)
    _, mixed = pn.windowed_attention(h, w, "p.", m, 0.0, pos, first)
    assert torch.allclose(mixed, 0.75 * v + 0.25 * first)


def test_plain_matrix_memory_by_hand():
    """One head, key size 1: with zi = zf = 0 and a cap far away, gi = 0 and gf = ln 1/2, so m stays 0 and the state is
    S_t = S_(t-1) / 2 + k v; the result is S q / (max(|n q|, 1) + 1e-6) before the head norm."""
    W = 3
    w = {"p.q": torch.tensor([[2.0, 0, 0]]), "p.k": torch.tensor([[0, 1.0, 0]]), "p.v": torch.tensor([[0, 0, 1.0], [0, 0, -1.0]]),
         "p.i": torch.zeros(1, W), "p.i.b": torch.zeros(1), "p.f": torch.zeros(1, W), "p.f.b": torch.zeros(1),
         "p.g": torch.zeros(2, W), "p.norm": torch.ones(2), "p.o": torch.eye(2)}
    h = torch.tensor([[1.0, 1.0, 3.0], [1.0, 2.0, 1.0]], dtype=D64)
    y = pn.matrix_memory(h, w, "p.", {"heads": 1, "dim": 1, "vdim": 2, "gate_cap": 1e6}, 0.0)
    # both rows: the two value columns are opposite, so the head norm leaves (+1, -1) times the sign; gate sigmoid(0) = 1/2
    assert torch.allclose(y, torch.tensor([[0.5, -0.5], [0.5, -0.5]], dtype=D64))
    # the un-normed ratio: token 2 has S = 3/2 + 2 * 1 = 3.5, n = 1/2 + 2 = 2.5, q = 2: 7 / (5 + 1e-6)
    w["p.norm"] = torch.tensor([1.0, 0.0])
    w["p.o"] = torch.tensor([[1.0, 0.0]])
    import plain_nukelix
    saved = plain_nukelix.rms
    plain_nukelix.rms = lambda x, eps: x
    try:
        y = pn.matrix_memory(h, w, "p.", {"heads": 1, "dim": 1, "vdim": 2, "gate_cap": 1e6}, 0.0)
    finally:
        plain_nukelix.rms = saved
    assert float(y[0, 0]) == pytest.approx(0.5 * 6.0 / (2.0 + 1e-6)) and float(y[1, 0]) == pytest.approx(0.5 * 7.0 / (5.0 + 1e-6))
    # a large forget bias keeps the first token: its value still shows a hundred tokens later
    T = 100
    hh = torch.zeros(T, W, dtype=D64)
    hh[:, 0] = 1.0
    hh[0] = torch.tensor([1.0, 1.0, 1.0])
    w["p.f.b"] = torch.tensor([8.0])
    plain_nukelix.rms = lambda x, eps: x
    try:
        far = pn.matrix_memory(hh, w, "p.", {"heads": 1, "dim": 1, "vdim": 2, "gate_cap": 10.0}, 0.0)
    finally:
        plain_nukelix.rms = saved
    assert float(far[-1, 0]) > 0.3


def test_plain_mixture_puts_the_weight_on_the_input():
    W = 4
    w = {"p.router": torch.tensor([[5.0, 0, 0, 0], [0, 5.0, 0, 0], [-5.0, -5.0, 0, 0]]), "p.shared.gate": torch.zeros(2, W),
         "p.shared.up": torch.zeros(2, W), "p.shared.down": torch.zeros(W, 2)}
    g = torch.Generator().manual_seed(2)
    for e in range(3):
        w[f"p.e{e}.gate"], w[f"p.e{e}.up"], w[f"p.e{e}.down"] = (torch.randn(3, W, generator=g), torch.randn(3, W, generator=g),
                                                                 torch.randn(W, 3, generator=g))
    h = torch.tensor([[1.0, 0.2, 0.5, -0.3]], dtype=D64)
    ids, wts = pn.route(h, w["p.router"], 2)
    assert ids[0].tolist() == [0, 1] and float(wts[0, 0]) == pytest.approx(1 / (1 + math.exp(-5.0))) and float(wts.sum()) > 1.5
    y = pn.mixture(h, w, "p.", {"router": {"experts": 3, "top": 2}, "shared": {"ff": 2}})
    by_input = sum(pn.gated_expert(wts[0, c] * h, w, f"p.e{int(ids[0, c])}.") for c in range(2))
    by_output = sum(wts[0, c] * pn.gated_expert(h, w, f"p.e{int(ids[0, c])}.") for c in range(2))
    assert torch.allclose(y, by_input) and not torch.allclose(y, by_output, atol=1e-4)


def test_plain_latent_attention_shares_one_rotated_key_part():
    cfg = nk.config(32, 50, [nk.layer("latent_attention", nk.latent(2, 4, 4, 3, 6, 5, 0.5, 100.0))])
    t = nk.draw_tensors(cfg, 4)
    h = torch.randn(6, 32, generator=torch.Generator().manual_seed(1), dtype=D64)
    m = cfg["layers"][0]["mixer"]
    base = pn.latent_attention(h, t, "l0.mix.", m, 1e-6, torch.arange(6))
    # the same tokens three places later: the shared key part turns with the queries' parts, so nothing changes ...
    later = pn.latent_attention(h, t, "l0.mix.", m, 1e-6, torch.arange(6) + 3)
    assert torch.allclose(base, later, atol=1e-12)
    # ... but the rows without the rotated part (its key rows zeroed) differ: the part takes part in the scores
    t2 = dict(t)
    t2["l0.mix.dkv"] = t["l0.mix.dkv"].clone()
    t2["l0.mix.dkv"][6:] = 0
    assert not torch.allclose(base, pn.latent_attention(h, t2, "l0.mix.", m, 1e-6, torch.arange(6)), atol=1e-6)


def test_plain_latent_space_form_is_the_same_attention():
    """Queries taken into the latent space and the values' map applied after the weighted sum: the same numbers."""
    cfg = nk.config(32, 50, [nk.layer("latent_attention", nk.latent(3, 6, 4, 5, 9, 7, 0.5, 100.0, (2.0, 8, 2.0, 1.0)))])
    t = nk.draw_tensors(cfg, 6)
    h = torch.randn(11, 32, generator=torch.Generator().manual_seed(2), dtype=D64)
    m = cfg["layers"][0]["mixer"]
    plain = pn.latent_attention(h, t, "l0.mix.", m, 1e-6, torch.arange(11))
    saved = pn.ROUND
    pn.ROUND = lambda x: x * 1.0                               # not the marker of exact arithmetic, and yet exact
    try:
        other = pn.latent_attention(h, t, "l0.mix.", m, 1e-6, torch.arange(11))
    finally:
        pn.ROUND = saved
    assert torch.allclose(plain, other, atol=1e-12)


# ---- the engine's host logic ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "chunks", "mixed"])
def test_host_logic_on_the_cpu_stand_in(name, mode, tmp_path, cpu_ops):
    cfg, lengths, page = nk.CASES[name]
    folder = nk.write_model(str(tmp_path / "m"), cfg, seed=3)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(lengths)}
    tensors = helpers.read_tensors(folder)
    ref = {rid: pn.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    steps = {"whole": helpers.trace_whole, "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=4)}[mode](reqs)
    runner = _runner(folder, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(lengths)
    assert _rel(got, ref) < 3e-4
    assert runner.cache.n_live == 0
    runner.cache.check()


def test_pages_behind_a_window_go_back_but_the_kept_first_tokens_stay(cpu_ops, tmp_path):
    """A windowed layer with kept first tokens gives back the pages between the kept tokens and the window, and only
    those: the request's block table keeps its first pages and its last ones."""
    cfg = nk.config(32, 60, [nk.layer("attention", nk.attention(2, 1, 8, 8, 0.4, window=6, keep_first=5, rotation=nk.rot(4, 50.0)))])
    folder = nk.write_model(str(tmp_path / "m"), cfg, seed=5)
    toks = helpers.random_tokens(41, 60, 3)
    ref = pn.forward(cfg, helpers.read_tensors(folder), toks).float()
    runner = _runner(folder, 4, 64, max_requests=1)
    steps = helpers.trace_chunks({"a": toks}, sizes=(9, 2, 7, 3))
    got = {}
    from kungfu_b200.engine import StepEntry
    runner.cache.add_request("a")
    at = 0
    for s in steps:
        e = s["entries"][0]
        out = runner.step([StepEntry("a", e["tokens"], e["want"])])
        for i, wpos in enumerate(e["want"]):
            got[("a", at + wpos)] = out[i].clone()
        at += len(e["tokens"])
    assert _rel(got, {"a": ref}) < 3e-4
    row = [int(p) for p in runner.cache.block_table(0, "a")[: -(-41 // 4)]]
    held = [i for i, p in enumerate(row) if p >= 0]
    # kept: tokens 0..4 -> pages 0 and 1; the window of the next query (position 41) reaches back to token 36 -> page 9
    assert held[:2] == [0, 1] and all(i >= 9 for i in held[2:]) and 10 in held and 5 not in held
    runner.cache.release("a")
    runner.cache.check()
