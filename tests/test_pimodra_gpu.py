"""Pimodra on the GPU against the plain implementation (tests/plain_pimodra.py, float64, whole sequences).

First the new kernels alone (norms in groups with and without the fused sum, the shift and the next norm; the activation
that norms powers; rotation, unit norm and filing of keys; the heads' mixing and gate; the softmax router), then every
mechanism alone as a one-layer model, then whole models through the step function in every way of cutting the work,
in 32-bit and in bfloat16; then window edges and far keys made to stand out, long decoding, used-again pages and slots,
generation through the engine, and the programs in bin/.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import pimodra_cases as pm
import plain_pimodra as pp

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 4e-2}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max()) / max(float(b.double().abs().max()), 1e-30)


# ---- the kernels alone -----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,groups", [(64, 2), (96, 1), (100, 5), (30, 3), (512, 8), (2304, 4), (320, 64)])
def test_group_norms_alone_and_fused(dtype, W, groups):
    from kungfu_b200 import ops
    tdt = DTYPES[dtype]
    tol = 2e-6 if dtype == "float32" else 1e-2
    g = torch.Generator().manual_seed(W + groups)
    T = 37
    x = 3.0 * torch.randn(T, W, generator=g)
    w1, w2 = (1 + 0.3 * torch.randn(W, generator=g)).to(tdt), (1 + 0.3 * torch.randn(W, generator=g)).to(tdt)
    shift = torch.randn(W, generator=g).to(tdt)
    out = torch.empty(T, W, dtype=tdt, device=DEV)
    ops.group_rmsnorm(x.to(DEV), w1.to(DEV), 1e-5, groups, out)
    assert _rel(out, pp.group_norm(x.double(), w1, 1e-5, groups)) < tol
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    some = torch.empty(4, W, dtype=tdt, device=DEV)
    ops.group_rmsnorm(x.to(DEV), w1.to(DEV), 1e-5, groups, some, rows.to(DEV))
    assert _rel(some, pp.group_norm(x.double()[rows.long()], w1, 1e-5, groups)) < tol
    # residual += norm(branch); next = norm(residual)
    res, branch = torch.randn(T, W, generator=g), 2.0 * torch.randn(T, W, generator=g)
    rd, nxt = res.to(DEV), torch.empty(T, W, dtype=tdt, device=DEV)
    ops.add_group_rmsnorm(branch.to(DEV), w1.to(DEV), 1e-5, groups, rd, next_weight=w2.to(DEV), next_eps=1e-4, next_out=nxt)
    ref = res.double() + pp.group_norm(branch.double(), w1, 1e-5, groups)
    assert _rel(rd, ref) < 2e-6 and _rel(nxt, pp.group_norm(ref, w2, 1e-4, groups)) < tol
    rd2 = res.to(DEV)
    ops.add_group_rmsnorm(branch.to(DEV), w1.to(DEV), 1e-5, groups, rd2)
    assert _rel(rd2, ref) < 2e-6
    # residual += a constant row; next = norm(residual)
    rd3 = res.to(DEV)
    ops.add_group_rmsnorm(None, None, 0.0, groups, rd3, shift=shift.to(DEV), next_weight=w2.to(DEV), next_eps=1e-5, next_out=nxt)
    ref3 = res.double() + shift.double()
    assert _rel(rd3, ref3) < 2e-6 and _rel(nxt, pp.group_norm(ref3, w2, 1e-5, groups)) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("I", [34, 96, 150, 1024, 9216])
def test_activation_that_norms_powers(dtype, I):
    from kungfu_b200 import ops
    g = torch.Generator().manual_seed(I)
    z = 1.5 * torch.randn(21, I, generator=g)
    coef = torch.tensor([0.8, -0.5, 0.4, 0.1]).to(DTYPES[dtype])
    out = torch.empty(21, I, dtype=DTYPES[dtype], device=DEV)
    ops.poly_norm(z.to(DEV), coef.to(DEV), 1e-5, out)
    assert _rel(out, pp.poly_norm(z.double(), coef, 1e-5)) < (3e-6 if dtype == "float32" else 1e-2)
    # each of the four numbers alone, so that none hides behind another
    for k in range(4):
        one = torch.zeros(4)
        one[k] = 1.0
        ops.poly_norm(z.to(DEV), one.to(DTYPES[dtype]).to(DEV), 1e-5, out)
        assert _rel(out, pp.poly_norm(z.double(), one, 1e-5)) < (3e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("E,G,keep,top", [(8, 2, 1, 2), (6, 1, 1, 3), (5, 1, 1, 1), (12, 3, 1, 4), (16, 4, 2, 4), (64, 8, 4, 7),
                                          (8, 4, 2, 3), (40, 40, 3, 2)])
def test_softmax_router_against_the_plain_choice(E, G, keep, top):
    from kungfu_b200 import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    T = 133
    logits = 2.0 * torch.randn(T, E, generator=g)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    w = torch.empty(T, top, device=DEV)
    ops.moe_route(logits.to(DEV), None, G, keep, top, 1.0, ids, w, score="softmax", group_rank="best", normalize=False)
    rid, rw = pp.route(logits.double(), E, top, G, keep)
    got = [dict(zip(a.tolist(), b.tolist())) for a, b in zip(ids.cpu(), w.cpu())]
    for t in range(T):
        want = dict(zip(rid[t].tolist(), rw[t].tolist()))
        assert set(got[t]) == set(want), t
        assert all(abs(got[t][e] - want[e]) < 1e-6 for e in want)
    assert float(w.sum(-1).max()) < 1.0 + 1e-5 and (top == E or float(w.sum(-1).min()) < 0.999)     # not renormalised


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,W,ff", [(1, 8, 2, 64, 32), (37, 6, 3, 100, 30), (300, 16, 4, 512, 256), (130, 3, 2, 200, 72)])
def test_silu_gated_experts_as_grouped_products(dtype, T, E, top, W, ff):
    from kungfu_b200 import ops
    import test_petanex_gpu as other
    st = other.FakeStep()
    tdt = DTYPES[dtype]
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(tdt)
    wgu = (torch.randn(E, 2 * ff, W, generator=g) / W ** 0.5 * 2).to(tdt)
    wd = (torch.randn(E, W, ff, generator=g) / ff ** 0.5).to(tdt)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    plan = ops.moe_plan(ids.to(DEV), E, st)
    h = torch.empty(T * top, ff, dtype=tdt, device=DEV)
    ops.moe_linear(x.to(DEV), plan, wgu.to(DEV), h, gather=True, gated=True, activation="silu")
    eo = torch.empty(T * top, W, device=DEV)
    ops.moe_linear(h, plan, wd.to(DEV), eo, gather=False)
    y = torch.empty(T, W, device=DEV)
    ops.moe_combine(eo, plan, wts.to(DEV), None, y)
    ref = torch.zeros(T, W, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            gu = wgu[e].double() @ x[t].double()
            hid = gu[:ff] * torch.sigmoid(gu[:ff]) * gu[ff:]
            if dtype == "bfloat16":
                hid = hid.to(torch.bfloat16).double()
            ref[t] += float(wts[t, j]) * (wd[e].double() @ hid)
    assert _rel(y, ref) < (2e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,P,window", [(4, 2, 16, 4, 9), (3, 3, 32, 16, None), (8, 2, 64, 64, 100), (4, 1, 64, 64, None),
                                            (8, 4, 128, 64, 70), (6, 3, 48, 8, 24), (40, 2, 64, 64, None)])
@pytest.mark.parametrize("own_decode_kernel", [True, False])
def test_every_query_head_over_every_value_head(dtype, H, G, d, P, window, own_decode_kernel, monkeypatch):
    """`paged_attention(value_split=G)`: H * G result heads from H query heads and G stored heads, on every kernel the step
    would choose (whole prompts, rows in the middle of a prompt, single decode rows with the keys in one part and cut
    into several; 40 heads over 2: tiles of heads that straddle two key heads, or the decode kernel without tensor cores).  The reference attends head by head with the keys of the query's head and the values of each."""
    import math
    import test_gpu_kernels as tk
    from kungfu_b200 import ops
    # decode rows: the kernel that owns all value heads of a tile of query heads, or the ordinary decode kernels
    monkeypatch.setattr(ops, "decode_value_split_kernel", own_decode_kernel)
    tdt = DTYPES[dtype]
    lens = [1, 37, 150, 70, 200, 1500]
    pages, table, ks, vs = tk._paged_setup(tdt, H, G, d, P, lens, seed=15)         # pages of G heads
    per = H // G
    scale = 1.0 / math.sqrt(d)
    g = torch.Generator().manual_seed(16)

    def run(rows, dec_rows, pre_rows):
        q = torch.randn(len(rows), H, d, generator=g).to(tdt)
        ctx = tk._Ctx(torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV),
                      torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV), table.to(DEV), dec_rows, pre_rows)
        out = torch.empty(len(rows), H * G * d, dtype=tdt, device=DEV)
        ops.paged_attention(q.view(len(rows), H * d).to(DEV), out, ctx, tk._View(pages.to(DEV), P), H * G, G * G, d, scale, 0.0,
                            window, value_split=G)
        got = out.view(len(rows), H * G, d).double().cpu()
        for i, (r, pos) in enumerate(rows):
            lo = max(0, pos - window + 1) if window else 0
            for gq in range(H):
                kh = gq // per
                a = torch.softmax((ks[r][lo:pos + 1, kh].double() @ q[i, gq].double()) * scale, 0)
                for c in range(G):
                    want = a @ vs[r][lo:pos + 1, c].double()
                    wide = (kh * G + c) * per + gq % per
                    err = float((got[i, wide] - want).abs().max()) / max(float(want.abs().max()), 1e-6)
                    assert err < (2e-5 if dtype == "float32" else 2e-2), (i, gq, c, err)

    # a whole prompt, the tail of another, and single rows of three requests in one step
    rows = [(1, p) for p in range(37)] + [(3, p) for p in range(50, 70)] + [(2, 149), (0, 0), (4, 199)]
    run(rows, [57, 58, 59], list(range(57)))
    run([(2, 149), (0, 0), (4, 199), (3, 69)], [0, 1, 2, 3], None)                 # a decode step
    run([(5, 1499), (0, 0), (5, 1200), (1, 36)], [0, 1, 2, 3], None)               # long rows: the keys cut into many parts
    run([(4, p) for p in range(200)], None, list(range(200)))                      # a long prompt alone


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dv,D,gate,mixed", [(4, 2, 24, 32, True, True), (3, 3, 12, 16, True, True), (4, 1, 64, 64, True, True),
                                                 (8, 4, 64, 128, True, True), (2, 2, 7, 16, True, True), (36, 2, 6, 16, False, True),
                                                 (112, 8, 8, 16, True, True), (5, 5, 16, 16, True, False), (3, 1, 5, 32, False, False)])
def test_heads_mixed_and_gated(dtype, H, G, dv, D, gate, mixed):
    """`head_mix_gate` alone: rows of 2 and 4 elements per thread, odd value sizes, 18 heads per value head (more than a
    thread sums at once), a mixing matrix too large for shared memory, no gate, no mixing, and a padding row."""
    from kungfu_b200 import ops
    import test_petanex_gpu as other
    st = other.FakeStep(rows=(6, 1, 4))
    T = st.n_rows
    tdt = DTYPES[dtype]
    g = torch.Generator().manual_seed(H * 100 + dv)
    per = H // G
    o = torch.randn(T, H * (G if mixed else 1), D, generator=g).to(tdt)
    mix = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).to(tdt) if mixed else None
    gcol0 = 8
    proj = torch.randn(T, gcol0 + H * dv + 4, generator=g)
    out = torch.full((T, H * dv), 7.0, dtype=tdt, device=DEV)
    ops.head_mix_gate(o.reshape(T, -1).to(DEV), None if mix is None else mix.to(DEV), proj.to(DEV) if gate else None, gcol0, H, G,
                      dv, D, out, st)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for h in range(H):
        if mixed:
            for gq in range(H):
                want[:, h] += float(mix[h, gq]) * o[:, ((gq // per) * G + h // per) * per + gq % per, :dv].double()
        else:
            want[:, h] = o[:, h, :dv].double()
    want = want.reshape(T, H * dv)
    if gate:
        want = want * torch.sigmoid(proj[:, gcol0:gcol0 + H * dv].double())
    want[-1] = 0                                              # the padding row
    assert _rel(out, want) < (3e-6 if dtype == "float32" else 1e-2)


# ---- the model through the step function -------------------------------------------------------------------------

def _runner(folder, dtype, page, max_tokens, max_requests=4, graphs=True, ctx=2048):
    from kungfu_b200 import api
    cfg, model = api.load_model(folder, dtype=dtype, device=DEV)
    return api.make_runner(cfg, model, dtype=dtype, device=DEV, page_size=page, max_tokens=max_tokens,
                           max_requests=max_requests, max_context=ctx, cuda_graphs=graphs)


def _plain(cfg, tensors, toks):
    """(exact logits, logits with the plain implementation rounding to bfloat16 where a 16-bit path may), both float32."""
    exact = pp.forward(cfg, tensors, toks).float()
    with pp.rounded_to_bfloat16():
        return exact, pp.forward(cfg, tensors, toks).float()


def _quantiles(errs):
    errs = sorted(errs)
    n = len(errs)
    return errs[n // 2], errs[min(n - 1, (n * 19) // 20)], errs[-1]


def _check(got, ref, tol, noisy=None):
    """32-bit: the largest difference of any logit against the largest logit, below `tol` at every place.  bfloat16: small
    random models amplify 8-bit rounding unevenly (a close call between two experts falls the other way, a sharp softmax
    moves), so the yardstick is the model itself: `noisy` holds the plain implementation's logits with its 16-bit roundings
    switched on.  Per place, the error is the root mean square of the differences against that of the place's logits; the
    median, the 95th percentile and the largest error of the framework must stay within twice those of the yardstick
    (with a floor of tol / 8 for models that rounding hardly moves)."""
    assert got
    if tol < 1e-2:
        scale = max(float(r.abs().max()) for r in ref.values())
        worst = max(float((row - ref[rid][pos]).abs().max()) for (rid, pos), row in got.items()) / scale
        assert worst < tol, f"rel err {worst:.3e}"
        return
    assert noisy is not None
    rel = lambda a, b: float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt())
    mine = _quantiles([rel(row, ref[rid][pos]) for (rid, pos), row in got.items()])
    yard = _quantiles([rel(noisy[rid][pos], ref[rid][pos]) for (rid, pos) in got])
    for m, y, what in zip(mine, yard, ("median", "95 %", "largest")):
        assert m < max(2.0 * y, tol / 8), f"rel err {what} {m:.3e}, rounding alone {y:.3e}"


ONE_LAYER = {
    # the heads' weights mixed over two value heads, values wider than keys, part of a head rotated, slow pairs stretched
    "attention": pm.config(64, 200, [pm.layer(pm.attention(4, 2, 16, 24, 0.9, window=50, rotation=pm.rot(8, 100.0, (2.0, 16, 4.0, 1.0))))], groups=2),
    # as many value heads as heads (every head's weights reach every value head), no window, no rotation
    "all_heads": pm.config(48, 200, [pm.layer(pm.attention(3, 3, 8, 12, 1.3))], groups=3),
    # one value head; tensor-core head sizes
    "one_value_head": pm.config(128, 200, [pm.layer(pm.attention(4, 1, 64, 64, 0.5, window=70, rotation=pm.rot(64, 10000.0, (4.0, 32, 8.0, 1.0))))], groups=1),
    "wide": pm.config(256, 200, [pm.layer(pm.attention(8, 4, 128, 64, 0.3, rotation=pm.rot(32, 1000.0)))], groups=4),
    "dense": pm.config(64, 200, [pm.layer(pm.attention(1, 1, 8, 8, 1.0), pm.dense(96))], groups=2),
    "moe": pm.config(64, 200, [pm.layer(pm.attention(1, 1, 8, 8, 1.0), pm.moe(8, 3, 32, groups=(4, 2)))], groups=4),
    "loop": pm.config(64, 200, [pm.layer(pm.attention(2, 1, 8, 8, 1.0, window=9), pm.dense(40))], groups=2, loop=(0, 1, 3)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mechanism_alone_as_a_one_layer_model(which, dtype, tmp_path):
    cfg = ONE_LAYER[which]
    folder = pm.write_model(str(tmp_path / "m"), cfg, seed=7)
    reqs = {"a": helpers.random_tokens(150, cfg["vocab"], 1), "b": helpers.random_tokens(9, cfg["vocab"], 2)}
    tensors = helpers.read_tensors(folder)
    both = {rid: _plain(cfg, tensors, toks) for rid, toks in reqs.items()}
    ref, noisy = {r: b[0] for r, b in both.items()}, {r: b[1] for r, b in both.items()}
    for steps in (helpers.trace_whole(reqs), helpers.trace_chunks(reqs), helpers.trace_decode_tail(reqs, 8)):
        runner = _runner(folder, dtype, 64, helpers.trace_max_tokens(steps, 64))
        _check(helpers.run_trace_with_runner(runner, steps), ref, TOL[dtype], noisy)


def test_residual_after_every_layer_run(tmp_path):
    """The 32-bit residual stream after each layer run, looped runs counted each time, against the plain one."""
    from kungfu_b200.engine import StepEntry
    cfg = pm.PM_A
    folder = pm.write_model(str(tmp_path / "m"), cfg, seed=11)
    toks = helpers.random_tokens(40, cfg["vocab"], 3)
    _, after = pp.forward(cfg, helpers.read_tensors(folder), toks, keep_layers=True)
    runner = _runner(folder, "float32", 4, 64, graphs=False)
    runner.cache.add_request("a")
    kept = []
    runner.model.after_layer = lambda i, x: kept.append(x[:len(toks)].detach().clone())
    try:
        runner.step([StepEntry("a", toks, [len(toks) - 1])])
    finally:
        runner.model.after_layer = None
    assert len(kept) == after.shape[0]
    for i, x in enumerate(kept):
        assert x.dtype == torch.float32 and _rel(x, after[i]) < 1e-4, i


NOISY = {}          # per model of the fixture below: request -> the plain implementation's logits with 16-bit roundings


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    cases = dict(pm.CASES)
    cases["E"] = (pm.PM_E, [3, 130, 64, 200, 65, 17], 64)
    for name, (cfg, lengths, page) in cases.items():
        folder = pm.write_model(str(tmp_path_factory.mktemp(name) / "m"), cfg, seed=21)
        reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(lengths)}
        tensors = helpers.read_tensors(folder)
        both = {rid: _plain(cfg, tensors, toks) for rid, toks in reqs.items()}
        out[name] = (folder, cfg, reqs, {r: b[0] for r, b in both.items()}, page)
        NOISY[name] = {r: b[1] for r, b in both.items()}
    return out


def _steps(mode, reqs):
    return {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_decode_tail(r, 32),
            "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=5)}[mode](reqs)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_modes_match_plain(models, name, mode, dtype):
    """Whole prompts, most of a prompt then token by token, portions of 2 to 11 tokens, and mixed batches of up to four
    unequal requests with pools so small that pages are used again."""
    from kungfu_b200 import ops
    folder, cfg, reqs, ref, page = models[name]
    steps = _steps(mode, reqs)
    runner = _runner(folder, dtype, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _check(got, ref, TOL[dtype], NOISY[name])
    ops.raise_on_device_error(torch.device(DEV))
    assert runner.cache.n_live == 0
    if mode == "mixed":
        assert all(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))


@pytest.mark.parametrize("name,page", [("A", 4), ("E", 64)])
def test_batch_of_unequal_requests_equals_each_alone(models, name, page):
    """32-bit: the logits of a request must not depend on what else is in its step."""
    from kungfu_b200.engine import StepEntry
    folder, cfg, reqs, ref, _ = models[name]
    runner = _runner(folder, "float32", page, 1024, graphs=False)
    alone = {}
    for rid, toks in reqs.items():
        runner.cache.add_request(rid)
        alone[rid] = runner.step([StepEntry(rid, toks, [len(toks) - 1])])[0].clone()
        runner.cache.release(rid)
    some = list(reqs)[:4]
    for rid in some:
        runner.cache.add_request(rid)
    together = runner.step([StepEntry(rid, reqs[rid], [len(reqs[rid]) - 1]) for rid in some]).clone()
    for i, rid in enumerate(some):
        scale = float(ref[rid].abs().max())
        assert float((together[i] - alone[rid]).abs().max()) / scale < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "E"])
def test_long_decoding_from_captured_graphs(models, name, dtype):
    """A short prompt and then 150 tokens one by one (the decode steps replay from a CUDA graph after the second); the
    windows of both models pass over decoded tokens only."""
    folder, cfg, _, _, page = models[name]
    toks = helpers.random_tokens(160, cfg["vocab"], 9)
    exact, noisy = _plain(cfg, helpers.read_tensors(folder), toks)
    steps = helpers.trace_decode_tail({"a": toks}, 150)
    runner = _runner(folder, dtype, page, 192)
    got = helpers.run_trace_with_runner(runner, steps)
    _check(got, {"a": exact}, TOL[dtype], {"a": noisy})
    assert any(s.get("graph") is not None for s in runner._graphs.values())


def _echo_model(folder, window, rotation, seed):
    """A one-layer model without a feed-forward in which token 250 + 2k + 1 "calls" token 250 + 2k: the keys' matrix is
    the queries' matrix behind a fixed shuffle of the input's elements (inside each group of the norm, whose weight is
    one), and the caller's embedding is the callee's shuffled the same way.  So the caller's query meets the callee's key
    with the largest score there is (unit vectors: the key size times `scale`), far above every other key's, its own
    included, while the two tokens' values differ: one key carries the row.  Two heads over two value heads, mixed."""
    cfg = pm.config(64, 300, [pm.layer(pm.attention(2, 2, 32, 16, 1.0, window=window, rotation=rotation))], groups=2)
    t = pm.draw_tensors(cfg, seed)
    shuffle = torch.cat([torch.roll(torch.arange(32), 5), 32 + torch.roll(torch.arange(32), 11)])
    t["l0.norm1"] = torch.ones_like(t["l0.norm1"])
    t["l0.mix.k"] = torch.zeros_like(t["l0.mix.q"])
    t["l0.mix.k"][:, shuffle] = t["l0.mix.q"]                       # W_k h = W_q (h taken in shuffled order)
    for callee in range(250, 300, 2):
        t["embed"][callee][shuffle] = t["embed"][callee + 1]         # the callee's row, shuffled, is the caller's
    from kungfu_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), t)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return cfg, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [40, 64, 100, 129])
def test_keys_just_inside_and_just_outside_a_window_stand_out(window, dtype, tmp_path):
    """Pairs of a callee and its caller are planted `window - 1` apart (the caller still sees the callee) and `window`
    apart (it no longer does), in the prompt and among the tokens decoded one by one, at page borders too.  The plain
    implementation itself shows that each planted key decides its row: replacing the callee changes the caller's row by a
    lot when it is inside the window and not at all when it is outside."""
    folder = str(tmp_path / "m")
    cfg, tensors = _echo_model(folder, window, pm.rot(8, 10000.0), seed=3)
    n = 3 * window + 140
    toks = [t % 250 for t in helpers.random_tokens(n, 250, 5)]
    plants = []                                   # (callee's place, caller's place, inside?)
    at, rare = 2, 250
    for k in range(8):
        inside = k % 2 == 0
        second = at + (window - 1 if inside else window)
        if second >= n:
            break
        toks[at], toks[second] = rare, rare + 1
        plants.append((at, second, inside))
        rare += 2
        at += window // 2 + 7 + (62 - at % 64 if k == 3 else 0)     # one plant starts right before a page border
    ref = pp.forward(cfg, tensors, toks)
    scale = float(ref.abs().max())
    for first, second, inside in plants:
        moved = list(toks)
        moved[first] = 7
        delta = float((pp.forward(cfg, tensors, moved)[second] - ref[second]).abs().max()) / scale
        assert (delta > 0.05) if inside else (delta == 0.0), (first, second, inside, delta)
    reqs = {"a": toks}
    noisy = _plain(cfg, tensors, toks)[1]
    tail = n - (plants[len(plants) // 2][0] + 1)              # decoding starts between the copies of a middle plant
    for steps in (helpers.trace_whole(reqs), helpers.trace_decode_tail(reqs, tail), helpers.trace_chunks(reqs)):
        runner = _runner(folder, dtype, 64, helpers.trace_max_tokens(steps, 64))
        got = helpers.run_trace_with_runner(runner, steps)
        _check(got, {"a": ref.float()}, TOL[dtype], {"a": noisy})
        if dtype == "float32":
            for first, second, inside in plants:
                assert float((got[("a", second)] - ref[second].float()).abs().max()) / scale < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_hundreds_of_tokens_back_carries_the_row(dtype, tmp_path):
    """No window, no rotation: a callee at place 3 (and others at page borders) and its caller 500 to 700 places later,
    in the prompt and in decoding.  Losing that one key among hundreds changes the row by far more than the tolerance."""
    folder = str(tmp_path / "m")
    cfg, tensors = _echo_model(folder, None, None, seed=4)
    n = 720
    toks = [t % 250 for t in helpers.random_tokens(n, 250, 6)]
    plants = [(3, 520), (63, 600), (64, 655), (0, 700), (128, 719)]
    for k, (a, b) in enumerate(plants):
        toks[a], toks[b] = 250 + 2 * k, 251 + 2 * k
    ref = pp.forward(cfg, tensors, toks)
    scale = float(ref.abs().max())
    for a, b in plants:
        moved = list(toks)
        moved[a] = 7
        assert float((pp.forward(cfg, tensors, moved)[b] - ref[b]).abs().max()) / scale > 0.05
    reqs = {"a": toks}
    noisy = _plain(cfg, tensors, toks)[1]
    for steps in (helpers.trace_whole(reqs), helpers.trace_decode_tail(reqs, 130), helpers.trace_chunks(reqs, sizes=(97, 2, 130, 31))):
        runner = _runner(folder, dtype, 64, helpers.trace_max_tokens(steps, 64))
        _check(helpers.run_trace_with_runner(runner, steps), {"a": ref.float()}, TOL[dtype], {"a": noisy})


def test_pages_of_a_finished_request_are_used_again_and_start_clean(models):
    """A pool of two pages per group and one request slot: requests follow one another through the same pages; each is
    cut in two portions, the first of two tokens."""
    from kungfu_b200.engine import StepEntry
    folder, cfg, reqs, ref, page = models["B"]
    runner = _runner(folder, "float32", page, 2 * 64, max_requests=1, graphs=False)
    for rid in ("r3", "r2", "r5", "r3"):
        toks = reqs[rid]
        runner.cache.add_request(rid)
        a = runner.step([StepEntry(rid, toks[:2], [0, 1])]).cpu()
        b = runner.step([StepEntry(rid, toks[2:], [len(toks) - 3])]).cpu()
        runner.cache.release(rid)
        scale = float(ref[rid].abs().max())
        assert float((a[0] - ref[rid][0]).abs().max()) / scale < TOL["float32"]
        assert float((a[1] - ref[rid][1]).abs().max()) / scale < TOL["float32"]
        assert float((b[0] - ref[rid][len(toks) - 1]).abs().max()) / scale < TOL["float32"]
    assert all(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_through_the_entry_point(models, dtype):
    """Greedy generation through Engine (scheduler, portions under a token budget, tokens drawn on the device, graphs)
    against the plain implementation's best token at every place, near ties aside."""
    import kungfu_b200
    from kungfu_b200.sampling import Sampling
    folder, cfg, reqs, _, page = models["E"]
    tensors = helpers.read_tensors(folder)
    eng = kungfu_b200.Engine(folder, dtype=dtype, device=DEV, ctx=512, batch=64, parallel=4, page_size=page,
                             max_tokens_in_cache=1024)
    prompts = [reqs["r1"], reqs["r0"], reqs["r3"], reqs["r5"], reqs["r2"]]
    outs = eng.generate(prompts, Sampling(temperature=0.0), max_tokens=12, ignore_eos=True)
    margin = 1e-3 if dtype == "float32" else 5e-2
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        seq = list(p)
        for tok in o:
            logits = pp.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > margin * float(logits.abs().max()):
                assert int(torch.argmax(logits)) == tok
            seq.append(tok)


def test_programs_in_bin(models, tmp_path):
    """bin/trace_run replays a trace of a Pimodra folder; bin/kungfu inspects the folder, completes a prompt and times
    the model."""
    folder, cfg, reqs, ref, page = models["A"]
    steps = helpers.trace_mixed(reqs, seed=2)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(helpers.trace_max_tokens(steps, 64))],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    at = {rid: 0 for rid in reqs}
    scale = max(float(r.abs().max()) for r in ref.values())
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                assert float(np.abs(rows[k] - ref[e["id"]][at[e["id"]] + w].numpy()).max()) / scale < TOL["float32"]
                k += 1
            at[e["id"]] += len(e["tokens"])
    kungfu = os.path.join(ROOT, "bin", "kungfu")
    p = subprocess.run([sys.executable, kungfu, "inspect", folder, "--json"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    doc = json.loads(p.stdout)
    assert doc["architecture"] == "Pimodra" and doc["layers"] == 4 and not doc["missing"] and not doc["unexpected"]
    assert len(doc["states"]) == 8                                # one cache per layer run: the looped stretch runs three times
    p = subprocess.run([sys.executable, kungfu, "generate", "--model", folder, "--ids", json.dumps(reqs["r1"]), "--max-tokens", "5",
                        "--dtype", "float32", "--ignore-eos", "--ctx", "256"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    gen = json.loads(p.stdout.strip().splitlines()[-1])["generated"]
    tensors = helpers.read_tensors(folder)
    seq = list(reqs["r1"])
    for tok in gen:
        logits = pp.forward(cfg, tensors, seq)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) > 1e-3 * float(logits.abs().max()):
            assert int(torch.argmax(logits)) == tok
        seq.append(tok)
    p = subprocess.run([sys.executable, kungfu, "bench", "--model", folder, "--pp", "40", "--tg", "6", "--reps", "1", "--ctx", "256"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "| Pimodra | bfloat16 | pp40 |" in p.stdout and "| Pimodra | bfloat16 | tg6 |" in p.stdout
