"""Nukelix on the GPU against the plain implementation (tests/plain_nukelix.py, float64, whole sequences).

First the new kernels alone (attention with kept first tokens and a sink on every attention kernel; q|k|v normed over the
whole projection, turned and filed; the matrix memory whole, in portions and token by token; expert weights on the input),
then every mechanism alone as a one-layer model, then whole models through the step function in every way of cutting the
work, in 32-bit and in bfloat16; then window edges, kept first tokens and far keys made to stand out, long decoding,
used-again pages and slots, generation through the engine, and the programs in bin/.
"""
import json
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

import helpers
import nukelix_cases as nk
import plain_nukelix as pn

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 4e-2}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max()) / max(float(b.double().abs().max()), 1e-30)


# ---- the kernels alone -----------------------------------------------------------------------------------------------

def _paged(keys, values, P, dtype):
    """keys [n, G, D], values [n, G, D] of ONE request filed into pages in a shuffled order; (pages, block table)."""
    n, G, D = keys.shape
    n_pages = -(-n // P)
    order = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(n))[:n_pages]
    pages = torch.zeros(n_pages + 3, 2, G, P, D)
    for j in range(n):
        pages[order[j // P], 0, :, j % P] = keys[j]
        pages[order[j // P], 1, :, j % P] = values[j]
    return pages.to(dtype).to(DEV), order.to(torch.int32).view(1, -1).to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,P,window,keep,sink", [
    (4, 2, 16, 4, 9, 3, True), (3, 3, 32, 16, 20, 0, True), (8, 2, 64, 64, 100, 10, True), (4, 1, 64, 64, None, 0, True),
    (4, 4, 128, 64, 70, 130, True), (2, 1, 64, 64, 40, 5, False), (6, 2, 24, 8, 5, 7, True), (16, 1, 128, 64, 129, 64, True)])
@pytest.mark.parametrize("fast", [True, False])
def test_attention_with_kept_first_tokens_and_a_sink(dtype, H, G, D, P, window, keep, sink, fast, monkeypatch):
    """Rows of a prompt portion in the middle of a request and single decode rows, on the tensor-core kernels and on the
    generic one, against the plain attention with the same mask and denominator."""
    from kungfu_b200 import ops
    monkeypatch.setattr(ops, "use_fast_attention", fast)
    g = torch.Generator().manual_seed(H * D + (window or 0))
    n = 300
    q = torch.randn(n, H, D, generator=g)
    k = torch.randn(n, G, D, generator=g)
    v = torch.randn(n, G, D, generator=g)
    tdt = DTYPES[dtype]
    q, k, v = (t.to(tdt).double() for t in (q, k, v))
    scale = 2.0 / D ** 0.5
    ref = pn.attend(q, k, v, scale, pn.visible(n, window, keep), sink)
    pages, table = _paged(k, v, P, tdt)
    for rows in (list(range(140, 300)), [299], [150], list(range(0, 70))):
        T = len(rows)
        single = T == 1
        ctx = types.SimpleNamespace(
            positions=torch.tensor(rows, dtype=torch.int32, device=DEV), row_req=torch.zeros(T, dtype=torch.int32, device=DEV),
            block_tables=[table], max_kv_len=rows[-1] + 1, n_rows=T, n_dec_rows=T if single else 0, n_pre_rows=0 if single else T,
            dec_rows=None, pre_rows=None, n_tiles=0, n_wide=0)
        if not single:
            ctx.pre_rows = torch.arange(T, dtype=torch.int32, device=DEV)
            bounds = list(range(0, T, 64))
            ctx.tile_row0 = torch.tensor(bounds, dtype=torch.int32, device=DEV)
            ctx.tile_nrows = torch.tensor([min(64, T - b) for b in bounds], dtype=torch.int32, device=DEV)
            ctx.n_tiles = len(bounds)
            wide = list(range(0, T, 128))
            ctx.wide_row0 = torch.tensor(wide, dtype=torch.int32, device=DEV)
            ctx.wide_nrows = torch.tensor([min(128, T - b) for b in wide], dtype=torch.int32, device=DEV)
            ctx.n_wide = len(wide)
        cache = types.SimpleNamespace(pages=pages, page_size=P, group=0, writes=True)
        out = torch.empty(T, H * D, dtype=tdt, device=DEV)
        ops.paged_attention(q[rows].to(tdt).reshape(T, H * D).to(DEV), out, ctx, cache, H, G, D, scale, 0.0, window,
                            keep_first=keep, sink=sink)
        torch.cuda.synchronize()
        assert _rel(out.view(T, H, D), ref[rows]) < (2e-5 if dtype == "float32" else 2e-2), (rows[0], T)


@pytest.mark.parametrize("H,G,D,window,keep,sink", [(4, 2, 64, 900, 70, True), (4, 1, 128, 500, 200, True), (2, 2, 64, None, 0, True),
                                                    (8, 2, 64, 700, 0, True), (4, 4, 256, 300, 64, False)])
@pytest.mark.parametrize("plan", [None, (4, 0), (3, 2), (8, 0)])
def test_long_contexts_whose_keys_are_cut_into_runs(H, G, D, window, keep, sink, plan, monkeypatch):
    """Short portions and single rows at a context of 1,500 tokens on the tensor-core kernels: the prompt kernel cuts a
    tile's keys into several runs (planned, and forced to 3, 4 and 8), the decode kernel into several splits; the kept
    tokens lie in the first run and the sink is counted once."""
    from kungfu_b200 import ops
    monkeypatch.setattr(ops, "prefill_plan_override", plan)
    slow_before = ops.fallback_count()
    g = torch.Generator().manual_seed(H * D + (window or 0))
    n, P = 1500, 64
    q, k, v = (torch.randn(n, h, D, generator=g).to(torch.bfloat16).double() for h in (H, G, G))
    q[:, :, :] *= 1.5                                               # sharp rows: a few keys carry each
    scale = 2.0 / D ** 0.5
    ref = pn.attend(q, k, v, scale, pn.visible(n, window, keep), sink)
    pages, table = _paged(k, v, P, torch.bfloat16)
    for rows in (list(range(1400, 1437)), list(range(1200, 1500)), [1499], [1024]):
        T = len(rows)
        single = T == 1
        ctx = types.SimpleNamespace(
            positions=torch.tensor(rows, dtype=torch.int32, device=DEV), row_req=torch.zeros(T, dtype=torch.int32, device=DEV),
            block_tables=[table], max_kv_len=rows[-1] + 1, n_rows=T, n_dec_rows=T if single else 0, n_pre_rows=0 if single else T,
            dec_rows=None, pre_rows=None, n_tiles=0, n_wide=0)
        if not single:
            ctx.pre_rows = torch.arange(T, dtype=torch.int32, device=DEV)
            bounds, wide = list(range(0, T, 64)), list(range(0, T, 128))
            ctx.tile_row0 = torch.tensor(bounds, dtype=torch.int32, device=DEV)
            ctx.tile_nrows = torch.tensor([min(64, T - b) for b in bounds], dtype=torch.int32, device=DEV)
            ctx.n_tiles = len(bounds)
            ctx.wide_row0 = torch.tensor(wide, dtype=torch.int32, device=DEV)
            ctx.wide_nrows = torch.tensor([min(128, T - b) for b in wide], dtype=torch.int32, device=DEV)
            ctx.n_wide = len(wide)
        cache = types.SimpleNamespace(pages=pages, page_size=P, group=0, writes=True)
        out = torch.empty(T, H * D, dtype=torch.bfloat16, device=DEV)
        ops.paged_attention(q[rows].to(torch.bfloat16).reshape(T, H * D).to(DEV), out, ctx, cache, H, G, D, scale, 0.0, window,
                            keep_first=keep, sink=sink)
        torch.cuda.synchronize()
        ops.raise_on_device_error(torch.device(DEV))
        assert _rel(out.view(T, H, D), ref[rows]) < 2e-2, (rows[0], T)
    assert ops.fallback_count() == slow_before                      # every launch ran a tensor-core kernel


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,W,ff", [(1, 8, 2, 64, 32), (37, 6, 3, 100, 30), (300, 16, 4, 512, 256), (130, 3, 3, 200, 72)])
def test_experts_with_the_weight_on_their_input(dtype, T, E, top, W, ff):
    from kungfu_b200.parts import RoutedExperts
    tdt = DTYPES[dtype]
    g = torch.Generator().manual_seed(T + E)
    w = {"p.router": (4.0 * torch.randn(E, W, generator=g) / W ** 0.5).to(torch.bfloat16)}
    for e in range(E):
        w[f"p.e{e}.gate"] = (torch.randn(ff, W, generator=g) / W ** 0.5).to(torch.bfloat16)
        w[f"p.e{e}.up"] = (torch.randn(ff, W, generator=g) / W ** 0.5).to(torch.bfloat16)
        w[f"p.e{e}.down"] = (torch.randn(W, ff, generator=g) / ff ** 0.5).to(torch.bfloat16)
    x = torch.randn(T, W, generator=g).to(tdt)
    ref = pn.mixture(x.double(), w, "p.", {"router": {"experts": E, "top": top}, "shared": None})
    gu = torch.stack([torch.cat([w[f"p.e{e}.gate"], w[f"p.e{e}.up"]]) for e in range(E)]).to(tdt).to(DEV)
    down = torch.stack([w[f"p.e{e}.down"] for e in range(E)]).to(tdt).to(DEV)
    part = RoutedExperts(w["p.router"].to(tdt).to(DEV), None, gu, down, top=top, scale=1.0, limit=0.0, score="sigmoid",
                         group_rank="best", normalize=False, activation="silu", weight_on="input")
    bufs = {}
    ctx = types.SimpleNamespace(act_dtype=tdt, buf=lambda tag, shape, dt: bufs.setdefault((tag, shape, dt), torch.empty(shape, dtype=dt, device=DEV)))
    y = part.forward(x.to(DEV), ctx)
    torch.cuda.synchronize()
    err = (y.double().cpu() - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()
    # a close call between two experts may fall the other way under 16-bit rounding of the router's input
    assert float(err.median()) < (1e-5 if dtype == "float32" else 2e-2) and float((err > 0.1).float().mean()) <= (0.0 if dtype == "float32" else 0.05)



def _step_ctx(rows_of_reqs, slots, pad_rows=0):
    """A hand-made step: request r has rows_of_reqs[r] consecutive rows and state slot slots[r] (an idle request slot has
    0 rows); `pad_rows` padding rows (request -1) at the end."""
    starts, row_req, at = [], [], 0
    for r, n in enumerate(rows_of_reqs):
        starts.append(at)
        row_req += [r] * n
        at += n
    row_req += [-1] * pad_rows
    bufs = {}
    return types.SimpleNamespace(
        n_reqs=len(rows_of_reqs), n_rows=len(row_req), row_req=torch.tensor(row_req, dtype=torch.int32, device=DEV),
        req_row_start=torch.tensor(starts, dtype=torch.int32, device=DEV), req_n_rows=torch.tensor(rows_of_reqs, dtype=torch.int32, device=DEV),
        req_state_slot=torch.tensor(slots, dtype=torch.int32, device=DEV),
        buf=lambda tag, shape, dt: bufs.setdefault((tag, tuple(shape), dt), torch.empty(shape, dtype=dt, device=DEV)))


@pytest.mark.parametrize("H,d,dv", [(2, 8, 12), (3, 40, 50), (1, 4, 4), (4, 64, 64), (2, 128, 32), (1, 200, 24), (2, 6, 7), (16, 128, 512)])
def test_matrix_memory_walk_from_earlier_states(H, d, dv):
    """Three requests with earlier tokens in their states (one with a large running maximum, one fresh), an idle request
    slot and two padding rows: results and states after a step of unequal portions, and after the same rows one by one.
    The last shape has more blocks (3 requests x 16 heads x 32 blocks of columns) than the GPU holds at a time, so blocks
    of one head run one after another: each must find the head's n as the step before left it."""
    from kungfu_b200 import ops
    g = torch.Generator().manual_seed(H * d + dv)
    rows = [37, 1, 0, 18]
    slots = [2, 0, -1, 3]
    T = sum(rows)
    cap = 9.0
    width = 2 * H * d + H * dv + 2 * H
    pad = (-width) % 4
    proj = torch.randn(T + 2, width + pad, generator=g)
    proj[:, 2 * H * d + H * dv:] *= 3.0                               # gates that reach the cap
    bi, bf = 0.5 * torch.randn(H, generator=g), 3.0 + torch.randn(H, generator=g)
    S0 = torch.randn(4, H, d, dv, generator=g)
    copies = -(-dv // 16)                                              # a copy of n per 16 value columns, then m
    m_at = copies * d
    n0 = torch.zeros(4, H, m_at + 4)
    n0[:, :, :m_at] = torch.randn(4, H, d, generator=g).repeat(1, 1, copies)
    n0[0, :, m_at] = 40.0                                              # a running maximum far from zero
    n0[2, :, m_at] = -3.0
    S0[3], n0[3] = 0.0, 0.0                                            # a fresh request
    q0, k0, v0, i0, f0 = 0, H * d, 2 * H * d, 2 * H * d + H * dv, 2 * H * d + H * dv + H

    def reference(r, row0, n, state):
        x = proj[row0:row0 + n].double()
        gi, gf = pn.memory_gates(x[:, i0:i0 + H] + bi.double(), x[:, f0:f0 + H] + bf.double(), cap)
        return pn.memory_walk(x[:, q0:q0 + H * d].view(n, H, d) * d ** -0.5, x[:, k0:k0 + H * d].view(n, H, d),
                              x[:, v0:v0 + H * dv].view(n, H, dv), gi, gf, state)

    for one_by_one in (False, True):
        S, nst = S0.clone().to(DEV), n0.clone().to(DEV)
        out = torch.zeros(T + 2, H * dv, device=DEV)
        if not one_by_one:
            ops.mlstm(proj.to(DEV), q0, k0, v0, i0, f0, bi.to(DEV), bf.to(DEV), cap, S, nst, out, H, d, dv, _step_ctx(rows, slots, 2))
        else:
            starts = [0, 37, 38, 38]
            for step in range(max(rows)):
                live = [r for r in range(4) if step < rows[r]]
                ctx = _step_ctx([1] * len(live), [slots[r] for r in live])
                pick = torch.tensor([starts[r] + step for r in live])
                o = torch.zeros(len(live), H * dv, device=DEV)
                ops.mlstm(proj[pick].contiguous().to(DEV), q0, k0, v0, i0, f0, bi.to(DEV), bf.to(DEV), cap, S, nst, o, H, d, dv, ctx)
                out[pick.to(DEV)] = o
        torch.cuda.synchronize()
        at = 0
        for r, n in enumerate(rows):
            if n == 0:
                continue
            sl = slots[r]
            ref, (Sr, nr, mr) = reference(r, at, n, (S0[sl], n0[sl, :, :d], n0[sl, :, m_at]))
            assert _rel(out[at:at + n].view(n, H, dv), ref) < 1e-4, (r, one_by_one)     # 32-bit sums over up to 200 rows of the state
            # the state in the stabiliser's own units: exp(m) S and exp(m) n are what the design defines
            grow = torch.exp(nst[sl, :, m_at].double().cpu() - mr)
            got_S = S[sl].double().cpu() * grow[:, None, None]
            assert _rel(got_S, Sr) < 2e-5 and float((nst[sl, :, m_at].cpu() - mr).abs().max()) < 1e-3
            for c in range(copies):                                    # every block's copy of n
                assert _rel(nst[sl, :, c * d:(c + 1) * d].double().cpu() * grow[:, None], nr) < 2e-5
            at += n
        assert float(out[T:].abs().max()) == 0.0 and torch.equal(S[1].cpu(), S0[1])          # padding rows, the idle slot


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,dk,dv,rot,interleaved,P", [(4, 2, 16, 24, 8, True, 4), (3, 3, 8, 8, 8, False, 8), (8, 2, 64, 64, 32, True, 64),
                                                           (2, 1, 20, 10, 0, False, 16), (5, 5, 10, 6, 6, True, 16), (4, 4, 128, 64, 128, False, 64)])
def test_projections_normed_over_all_heads_turned_mixed_and_filed(dtype, nh, nkv, dk, dv, rot, interleaved, P):
    """q|k|v with biases -> the norms over the whole projections, rotation in either pairing, value mixing in both roles ->
    q rows and the pages, for two requests in the middle of their sequences and a padding row."""
    from kungfu_b200 import ops
    tdt = DTYPES[dtype]
    tol = 1e-5 if dtype == "float32" else 1e-2
    g = torch.Generator().manual_seed(nh * dk + dv)
    positions = [5, 6, 7, 8, 9, 10, 11, 30, 0]
    row_req = [0] * 7 + [1, -1]
    T = len(positions)
    D = ops.attention_head_size(max(dk, dv))
    C = (nh + nkv) * dk + nkv * dv
    ld = C + 4 + (-C) % 4
    proj = torch.randn(T, ld, generator=g)
    bias = (0.3 * torch.randn(C, generator=g)).to(tdt)
    wq, wk = (1 + 0.3 * torch.randn(nh * dk, generator=g)).to(tdt), (1 + 0.3 * torch.randn(nkv * dk, generator=g)).to(tdt)
    lam = torch.tensor([0.35]).to(tdt)
    first = torch.randn(T, nkv * dv, generator=g)
    freqs = pn.plain_frequencies({"base": 50.0, "dims": max(rot, 2)})[: rot // 2]
    ang = torch.tensor(positions, dtype=torch.float64)[:, None] * freqs[None, :]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    n_pages = 2 * (40 // P + 2)
    table = torch.arange(n_pages, dtype=torch.int32).view(2, -1)
    table = table.flip(1).contiguous().to(DEV)
    ctx = types.SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                                row_req=torch.tensor(row_req, dtype=torch.int32, device=DEV), block_tables=[table])
    x = proj[:, :C].double() + bias.double()
    q = pn.rms(x[:, :nh * dk], 1e-5) * wq.double()
    k = pn.rms(x[:, nh * dk:(nh + nkv) * dk], 1e-5) * wk.double()
    v = x[:, (nh + nkv) * dk:]
    pos_t = torch.tensor(positions)
    q = pn.rotate(q.view(T, nh, dk), pos_t, freqs, rot, interleaved, 1.25)
    k = pn.rotate(k.view(T, nkv, dk), pos_t, freqs, rot, interleaved, 1.25)
    for mode in (0, 1, 2):
        pages = torch.full((n_pages, 2, nkv, P, D), 7.0, dtype=tdt, device=DEV)
        cache = types.SimpleNamespace(pages=pages, page_size=P, group=0, writes=True)
        q_out = torch.full((T, nh * D), 7.0, dtype=tdt, device=DEV)
        shared = first.clone().to(DEV)
        ops.rownorm_rope_append(proj.to(DEV), 0, bias.to(DEV), wq.to(DEV), wk.to(DEV), 1e-5, cos if rot else None, sin if rot else None,
                                rot, interleaved, 1.25, nh, nkv, dk, dv, ctx, cache, q_out, v_mix=lam.to(DEV) if mode == 2 else None,
                                v_shared=shared if mode else None, v_mode=mode)
        torch.cuda.synchronize()
        want_v = v if mode != 2 else (1 - float(lam)) * v + float(lam) * first.double()
        qo = q_out.view(T, nh, D)
        assert _rel(qo[:8, :, :dk], q[:8]) < tol and float(qo[:8, :, dk:].abs().max() if D > dk else 0.0) == 0.0
        assert float(qo[8].abs().max()) == 0.0                          # the padding row's queries are zero
        for t in range(8):
            page = int(table[row_req[t], positions[t] // P])
            kk, vv = pages[page, 0, :, positions[t] % P], pages[page, 1, :, positions[t] % P]
            assert _rel(kk[:, :dk], k[t]) < tol and _rel(vv[:, :dv], want_v[t].view(nkv, dv)) < tol
            assert float(kk[:, dk:].abs().max() if D > dk else 0.0) == 0.0 and float(vv[:, dv:].abs().max() if D > dv else 0.0) == 0.0
        if mode == 1:
            assert _rel(shared[:8], v[:8]) < 1e-6                       # the first mixing layer leaves its values for the others


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,W", [(5, 64), (300, 512), (37, 100), (260, 2048)])
def test_sum_norm_and_copy_in_one_kernel(dtype, T, W):
    from kungfu_b200 import ops
    tdt = DTYPES[dtype]
    g = torch.Generator().manual_seed(T + W)
    res, branch = torch.randn(T, W, generator=g), 2.0 * torch.randn(T, W, generator=g)
    w = (1 + 0.3 * torch.randn(W, generator=g)).to(tdt)
    rd, copy = res.to(DEV), torch.empty(T, W, dtype=tdt, device=DEV)
    ops.add_rmsnorm(branch.to(DEV), w.to(DEV), 1e-5, False, rd, copy_out=copy)
    ref = res.double() + pn.rms(branch.double(), 1e-5) * w.double()
    assert _rel(rd, ref) < 2e-6 and _rel(copy, ref) < (2e-6 if dtype == "float32" else 1e-2)


def test_head_norm_with_one_weight_vector_per_head():
    from kungfu_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, H, dv = 9, 3, 20
    o, gate = torch.randn(T, H * dv, generator=g), torch.randn(T, H * dv + 8, generator=g)
    w = 1 + 0.3 * torch.randn(H * dv, generator=g)
    out = torch.empty(T, H * dv, device=DEV)
    ops.head_norm_gate(o.to(DEV), w.to(DEV), 1e-5, gate.to(DEV), 8, "sigmoid", out, H, dv)
    ref = (pn.rms(o.double().view(T, H, dv), 1e-5).reshape(T, H * dv) * w.double()) * torch.sigmoid(gate[:, 8:].double())
    assert _rel(out, ref) < 1e-5
    shared = 1 + 0.3 * torch.randn(dv, generator=g)
    ops.head_norm_gate(o.to(DEV), shared.to(DEV), 1e-5, gate.to(DEV), 8, "sigmoid", out, H, dv)
    ref = (pn.rms(o.double().view(T, H, dv), 1e-5) * shared.double()).reshape(T, H * dv) * torch.sigmoid(gate[:, 8:].double())
    assert _rel(out, ref) < 1e-5


# ---- models ------------------------------------------------------------------------------------------------------------

def _runner(folder, dtype, page, max_tokens, max_requests=4, graphs=True, ctx=2048):
    from kungfu_b200 import api
    cfg, model = api.load_model(folder, dtype=dtype, device=DEV)
    return api.make_runner(cfg, model, dtype=dtype, device=DEV, page_size=page, max_tokens=max_tokens,
                           max_requests=max_requests, max_context=ctx, cuda_graphs=graphs)


def _plain(cfg, tensors, toks):
    """(exact logits, logits with the plain implementation rounding to bfloat16 where a 16-bit path may), both float32."""
    exact = pn.forward(cfg, tensors, toks).float()
    with pn.rounded_to_bfloat16():
        return exact, pn.forward(cfg, tensors, toks).float()


def _quantiles(errs):
    errs = sorted(errs)
    n = len(errs)
    return errs[n // 2], errs[min(n - 1, (n * 19) // 20)], errs[-1]


def _check(got, ref, tol, noisy=None, tails=True):
    """32-bit: the largest difference of any logit against the largest logit, below `tol` at every place.  bfloat16: the
    yardstick is the model itself: `noisy` holds the plain implementation's logits with its 16-bit roundings switched on
    (the latent attention evaluated in the latent space, as a path that caches the latent alone has to).  The median of
    the framework's per-place errors must stay within twice the yardstick's, the 95th percentile and the largest error
    within three times (single events, a close call between two experts that falls the other way, decide those; `tails`
    False leaves them out for the model whose norms run over six elements), with a floor of tol / 8."""
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
    for m, y, what, factor in zip(mine, yard, ("median", "95 %", "largest"), (2.0, 3.0, 3.0)):
        if what == "median" or tails:
            assert m < max(factor * y, tol / 8), f"rel err {what} {m:.3e}, rounding alone {y:.3e}"


ONE_LAYER = {
    # values wider than keys, part of a head turned in interleaved pairs, frequencies rescaled, kept tokens, the sink
    "windowed": nk.config(64, 200, [nk.layer("attention", nk.attention(4, 2, 16, 24, 0.3, window=50, keep_first=6,
                                                                         rotation=nk.rot(8, 100.0, (3.0, 1.0, 4.0, 64))))]),
    # the same kind without a mask and without rotation: every earlier token and the sink
    "sink_only": nk.config(48, 200, [nk.layer("attention", nk.attention(3, 3, 8, 12, 0.5))]),
    # values mixed: the second layer takes the first one's
    "mixed_values": nk.config(64, 200, [nk.layer("attention", nk.attention(2, 2, 8, 8, 0.4, window=30, keep_first=2, v_mix=True)),
                                        nk.layer("attention", nk.attention(4, 2, 16, 8, 0.3, window=9, keep_first=0, v_mix=True))]),
    # tensor-core head sizes, a window longer than a page
    "windowed_wide": nk.config(128, 200, [nk.layer("attention", nk.attention(6, 2, 64, 64, 0.1, window=70, keep_first=12,
                                                                              rotation=nk.rot(64, 10000.0, (4.0, 1.0, 4.0, 32))))]),
    "side_by_side": nk.config(64, 200, [nk.layer("parallel", nk.parallel(nk.left(4, 2, 16, 8, 0.3, nk.rot(16, 100.0)), 2, 8, 12, 8.0, 0.7, 1.3))]),
    "memory_wide": nk.config(128, 200, [nk.layer("parallel", nk.parallel(nk.left(2, 1, 64, 64, 0.1, nk.rot(32, 1000.0)), 3, 40, 50, 14.0, 0.2, 1.5))]),
    "latent": nk.config(64, 200, [nk.layer("latent_attention", nk.latent(3, 8, 4, 6, 20, 12, 0.4, 1000.0, (2.0, 16, 4.0, 1.0)))]),
    "latent_wide": nk.config(256, 200, [nk.layer("latent_attention", nk.latent(20, 32, 16, 24, 100, 48, 0.1, 10000.0))]),
    # a latent whose stored head is above the largest the tensor-core kernels take: the generic kernel in both element types
    "latent_huge": nk.config(128, 200, [nk.layer("latent_attention", nk.latent(2, 16, 8, 12, 262, 20, 0.2, 100.0))]),
    "moe": nk.config(64, 200, [nk.layer("attention", nk.attention(1, 1, 8, 8, 0.5), nk.moe(8, 3, 32, shared=16))]),
    "moe_one": nk.config(64, 200, [nk.layer("attention", nk.attention(1, 1, 8, 8, 0.5), nk.moe(5, 1, 40))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mechanism_alone_as_a_one_layer_model(which, dtype, tmp_path):
    cfg = ONE_LAYER[which]
    folder = nk.write_model(str(tmp_path / "m"), cfg, seed=7, sharp=1.5)
    reqs = {"a": helpers.random_tokens(150, cfg["vocab"], 1), "b": helpers.random_tokens(9, cfg["vocab"], 2)}
    tensors = helpers.read_tensors(folder)
    both = {rid: _plain(cfg, tensors, toks) for rid, toks in reqs.items()}
    ref, noisy = {r: b[0] for r, b in both.items()}, {r: b[1] for r, b in both.items()}
    for steps in (helpers.trace_whole(reqs), helpers.trace_chunks(reqs), helpers.trace_decode_tail(reqs, 8)):
        runner = _runner(folder, dtype, 64, helpers.trace_max_tokens(steps, 64))
        _check(helpers.run_trace_with_runner(runner, steps), ref, TOL[dtype], noisy)


def test_residual_after_every_layer(tmp_path):
    """The 32-bit residual stream after each layer against the plain one."""
    from kungfu_b200.engine import StepEntry
    cfg = nk.NK_A
    folder = nk.write_model(str(tmp_path / "m"), cfg, seed=11)
    toks = helpers.random_tokens(40, cfg["vocab"], 3)
    after = pn.residuals(cfg, helpers.read_tensors(folder), toks)
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
    cases = dict(nk.CASES)
    cases["E"] = (nk.NK_E, [3, 130, 64, 200, 65, 17], 64)
    for name, (cfg, lengths, page) in cases.items():
        folder = nk.write_model(str(tmp_path_factory.mktemp(name) / "m"), cfg, seed=21)
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
    unequal requests with pools so small that pages and state slots are used again."""
    from kungfu_b200 import ops
    folder, cfg, reqs, ref, page = models[name]
    steps = _steps(mode, reqs)
    runner = _runner(folder, dtype, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _check(got, ref, TOL[dtype], NOISY[name], tails=name != "D")
    ops.raise_on_device_error(torch.device(DEV))
    assert runner.cache.n_live == 0
    if mode == "mixed":
        assert any(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))
        assert len(reqs) > runner.cache.max_requests           # state slots served more requests than there are slots


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
    windows of both models pass over decoded tokens only, and the memories carry their state through 150 steps."""
    folder, cfg, _, _, page = models[name]
    toks = helpers.random_tokens(160, cfg["vocab"], 9)
    exact, noisy = _plain(cfg, helpers.read_tensors(folder), toks)
    steps = helpers.trace_decode_tail({"a": toks}, 150)
    runner = _runner(folder, dtype, page, 192)
    got = helpers.run_trace_with_runner(runner, steps)
    _check(got, {"a": exact}, TOL[dtype], {"a": noisy})
    assert any(s.get("graph") is not None for s in runner._graphs.values())


def _echo_model(folder, kind, window, keep, rotation, seed):
    """A one-layer model without a feed-forward in which token 250 + 2k + 1 "calls" token 250 + 2k: the keys' matrix is
    the queries' matrix behind a fixed shuffle of the input's elements, the caller's embedding is the callee's shuffled
    the same way, biases are zero and both norm weights are one.  So the caller's normed query equals the callee's normed
    key and meets it with the largest score there is, far above every other key's, its own included, while the two
    tokens' values differ: one key carries the row.  `kind` 'attention': the windowed mixer; 'parallel': the attention
    beside a memory (scaled down so that the attention shows)."""
    if kind == "attention":
        cfg = nk.config(64, 300, [nk.layer("attention", nk.attention(2, 2, 32, 16, 0.5, window=window, keep_first=keep, rotation=rotation))])
        p = "l0.mix."
    else:
        cfg = nk.config(64, 300, [nk.layer("parallel", nk.parallel(nk.left(2, 2, 32, 16, 0.5, rotation), 2, 8, 8, 10.0, 1.0, 0.05))])
        p = "l0.mix.left."
    t = nk.draw_tensors(cfg, seed)
    shuffle = torch.cat([torch.roll(torch.arange(32), 5), 32 + torch.roll(torch.arange(32), 11)])
    t[p + "k"] = torch.zeros_like(t[p + "q"])
    t[p + "k"][:, shuffle] = t[p + "q"]                              # W_k h = W_q (h taken in shuffled order)
    for n in ("q.b", "k.b"):
        t[p + n] = torch.zeros_like(t[p + n])
    for n in ("q.norm", "k.norm"):
        t[p + n] = torch.ones_like(t[p + n])
    for callee in range(250, 300, 2):
        t["embed"][callee][shuffle] = t["embed"][callee + 1]         # the callee's row, shuffled, is the caller's
    nk.write_tensors(folder, cfg, t)
    return cfg, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep", [(40, 3), (64, 64), (100, 17), (129, 0)])
def test_keys_at_the_window_edge_and_among_the_kept_first_tokens_stand_out(window, keep, dtype, tmp_path):
    """Pairs of a callee and its caller are planted `window - 1` apart (the caller still sees the callee) and `window`
    apart (it no longer does), in the prompt and among the tokens decoded one by one, at page borders too; and callees
    at the last kept place (seen from far beyond the window) and at the first place that is not kept (not seen).  The
    plain implementation itself shows that each planted key decides its row."""
    folder = str(tmp_path / "m")
    cfg, tensors = _echo_model(folder, "attention", window, keep, nk.rot(8, 10000.0), seed=3)
    n = 3 * window + 140
    toks = [t % 250 for t in helpers.random_tokens(n, 250, 5)]
    plants = []                                   # (callee's place, caller's place, seen?)
    rare = 250
    if keep:
        for callee, caller, seen in ((keep - 1, keep - 1 + 2 * window + 9, True), (keep, keep + 2 * window + 30, False)):
            toks[callee], toks[caller] = rare, rare + 1
            plants.append((callee, caller, seen))
            rare += 2
    at = keep + 2
    for k in range(8):
        inside = k % 2 == 0
        second = at + (window - 1 if inside else window)
        if second >= n or any(second == c for _, c, _ in plants):
            break
        toks[at], toks[second] = rare, rare + 1
        plants.append((at, second, inside))
        rare += 2
        at += window // 2 + 7 + (62 - at % 64 if k == 3 else 0)     # one plant starts right before a page border
    ref = pn.forward(cfg, tensors, toks)
    scale = float(ref.abs().max())
    for first, second, seen in plants:
        moved = list(toks)
        moved[first] = 7
        delta = float((pn.forward(cfg, tensors, moved)[second] - ref[second]).abs().max()) / scale
        assert (delta > 0.05) if seen else (delta == 0.0), (first, second, seen, delta)
    reqs = {"a": toks}
    noisy = _plain(cfg, tensors, toks)[1]
    middle = sorted(p[0] for p in plants)[len(plants) // 2]
    tail = n - (middle + 1)                                    # decoding starts between the copies of a middle plant
    for steps in (helpers.trace_whole(reqs), helpers.trace_decode_tail(reqs, tail), helpers.trace_chunks(reqs)):
        runner = _runner(folder, dtype, 64, helpers.trace_max_tokens(steps, 64))
        got = helpers.run_trace_with_runner(runner, steps)
        _check(got, {"a": ref.float()}, TOL[dtype], {"a": noisy})
        if dtype == "float32":
            for first, second, seen in plants:
                assert float((got[("a", second)] - ref[second].float()).abs().max()) / scale < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_hundreds_of_tokens_back_carries_the_row(dtype, tmp_path):
    """The attention beside a memory, no window: a callee at place 3 (and others at page borders) and its caller 500 to
    700 places later, in the prompt and in decoding.  Losing that one key among hundreds changes the row by far more
    than the tolerance."""
    folder = str(tmp_path / "m")
    cfg, tensors = _echo_model(folder, "parallel", None, 0, None, seed=4)
    n = 720
    toks = [t % 250 for t in helpers.random_tokens(n, 250, 6)]
    plants = [(3, 520), (63, 600), (64, 655), (0, 700), (128, 719)]
    for k, (a, b) in enumerate(plants):
        toks[a], toks[b] = 250 + 2 * k, 251 + 2 * k
    ref = pn.forward(cfg, tensors, toks)
    scale = float(ref.abs().max())
    for a, b in plants:
        moved = list(toks)
        moved[a] = 7
        assert float((pn.forward(cfg, tensors, moved)[b] - ref[b]).abs().max()) / scale > 0.05
    reqs = {"a": toks}
    noisy = _plain(cfg, tensors, toks)[1]
    for steps in (helpers.trace_whole(reqs), helpers.trace_decode_tail(reqs, 130), helpers.trace_chunks(reqs, sizes=(97, 2, 130, 31))):
        runner = _runner(folder, dtype, 64, helpers.trace_max_tokens(steps, 64))
        _check(helpers.run_trace_with_runner(runner, steps), {"a": ref.float()}, TOL[dtype], {"a": noisy})


def test_a_memory_remembers_its_first_token_and_a_lost_state_shows(tmp_path):
    """A memory whose forget gates stay near one: the first token still moves the row 300 tokens later (the plain
    implementation says by how much), through portions and single tokens; zeroing the request's state slot between two
    steps moves the logits by far more than the tolerance."""
    from kungfu_b200.engine import StepEntry
    cfg = nk.config(64, 200, [nk.layer("parallel", nk.parallel(nk.left(1, 1, 8, 8, 0.3), 2, 16, 16, 13.0, 0.05, 1.5))])
    folder = str(tmp_path / "m")
    t = nk.draw_tensors(cfg, 8)
    t["l0.mix.right.f.b"] = torch.full_like(t["l0.mix.right.f.b"], 7.0)
    nk.write_tensors(folder, cfg, t)
    toks = helpers.random_tokens(320, 200, 4)
    ref = pn.forward(cfg, t, toks)
    scale = float(ref.abs().max())
    moved = list(toks)
    moved[0] = (toks[0] + 1) % 200
    assert float((pn.forward(cfg, t, moved)[300:] - ref[300:]).abs().max()) / scale > 0.02
    for steps in (helpers.trace_whole({"a": toks}), helpers.trace_decode_tail({"a": toks}, 40), helpers.trace_chunks({"a": toks})):
        runner = _runner(folder, "float32", 64, 384)
        _check(helpers.run_trace_with_runner(runner, steps), {"a": ref.float()}, TOL["float32"])
    runner = _runner(folder, "float32", 64, 384, graphs=False)
    runner.cache.add_request("a")
    runner.step([StepEntry("a", toks[:200], [])])
    for store in runner.cache.storage[0][1:]:
        store.zero_()                                            # the memory's two states (the pages come first)
    out = runner.step([StepEntry("a", toks[200:], [119])])
    assert float((out[0].cpu() - ref[319].float()).abs().max()) / scale > 20 * TOL["float32"]


def test_pages_and_slots_of_finished_requests_are_used_again_and_start_clean(models):
    """A pool of two pages per group and ONE state slot: requests follow one another through the same pages and the same
    slot of the memories; each is cut in two portions, the first of two tokens."""
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
    assert any(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))


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
            logits = pn.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > margin * float(logits.abs().max()):
                assert int(torch.argmax(logits)) == tok
            seq.append(tok)


def test_programs_in_bin(models, tmp_path):
    """bin/trace_run replays a trace of a Nukelix folder; bin/kungfu inspects the folder, completes a prompt and times
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
    assert doc["architecture"] == "Nukelix" and doc["layers"] == 4 and not doc["missing"] and not doc["unexpected"]
    assert len(doc["states"]) == 4
    p = subprocess.run([sys.executable, kungfu, "generate", "--model", folder, "--ids", json.dumps(reqs["r1"]), "--max-tokens", "5",
                        "--dtype", "float32", "--ignore-eos", "--ctx", "256"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    gen = json.loads(p.stdout.strip().splitlines()[-1])["generated"]
    tensors = helpers.read_tensors(folder)
    seq = list(reqs["r1"])
    for tok in gen:
        logits = pn.forward(cfg, tensors, seq)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) > 1e-3 * float(logits.abs().max()):
            assert int(torch.argmax(logits)) == tok
        seq.append(tok)
    p = subprocess.run([sys.executable, kungfu, "bench", "--model", folder, "--pp", "40", "--tg", "6", "--reps", "1", "--ctx", "256"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
