"""A slow CPU stand-in for `kungfu_b200.ops`, for tests on machines without a GPU.

It lets the engine's host logic (metadata, block tables, page reuse, scheduling) be checked against
the plain implementation without any kernel.  It is test equipment: the package has no CPU path and
never imports this file.  Each function mirrors the contract of the kernel of the same name.
"""
from __future__ import annotations

import math

import torch


def _act(name, x):
    if name == "gelu_tanh":
        return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    if name == "gelu_erf":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    return x * torch.sigmoid(x)


class CpuOps:
    def check_attention_sizes(self, nh, nkv, d, largest=256):
        assert nh % nkv == 0 and d % 2 == 0 and d <= largest

    def embed(self, tokens, table, scale, out):
        out.copy_(table.float()[tokens.long()] * torch.tensor(scale, dtype=torch.float32))

    def rmsnorm(self, x, weight, eps, plus_one, out, rows=None):
        xs = x if rows is None else x[rows.long()]
        inv = torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps)
        g = weight.float() + (1.0 if plus_one else 0.0)
        out.copy_((xs * inv * g).to(out.dtype))

    def add_rmsnorm(self, branch, weight, eps, plus_one, residual, *, next_weight=None, next_eps=0.0,
                    next_plus_one=False, next_out=None, copy_out=None):
        inv = torch.rsqrt(branch.pow(2).mean(-1, keepdim=True) + eps)
        residual.add_(branch * inv * (weight.float() + (1.0 if plus_one else 0.0)))
        if copy_out is not None:
            copy_out.copy_(residual.to(copy_out.dtype))
        if next_out is not None:
            self.rmsnorm(residual, next_weight, next_eps, next_plus_one, next_out)

    def add(self, a, x):
        x.add_(a)

    def linear(self, x, weight, out, softcap=0.0):
        y = x.float() @ weight.float().T
        if softcap > 0:
            y = softcap * torch.tanh(y / softcap)
        out.copy_(y.to(out.dtype))

    def linear_gated(self, x, w_gate_up, out, activation, ctx, limit=0.0):
        I = out.shape[1]
        gu = x.float() @ w_gate_up.float().T
        if activation == "clamped_swish":
            out.copy_(self._clamped(gu[:, :I], gu[:, I:], limit).to(out.dtype))
        else:
            out.copy_((_act(activation, gu[:, :I]) * gu[:, I:]).to(out.dtype))

    @staticmethod
    def _clamped(g, u, limit):
        g = torch.clamp(g, max=limit)
        u = torch.clamp(u, min=-limit, max=limit)
        return g * torch.sigmoid(1.702 * g) * (u + 1.0)

    def rope_table(self, positions, inv_freq, cos, sin):
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos.copy_(torch.cos(ang))
        sin.copy_(torch.sin(ang))

    def linear_rope_kv_append(self, x, wqkv, cos, sin, rot, nh, nkv, d, ctx, cache, q_out):
        return False                                   # no fused product here: the caller runs linear and rope_kv_append

    def rope_kv_append(self, qkv, cos, sin, rot, nh, nkv, d, ctx, cache, q_out):
        T = qkv.shape[0]
        q = qkv[:, :nh * d].view(T, nh, d).clone()
        k = qkv[:, nh * d:(nh + nkv) * d].view(T, nkv, d).clone()
        v = qkv[:, (nh + nkv) * d:].view(T, nkv, d)
        if rot:
            half = rot // 2
            c, s = cos[:, None, :], sin[:, None, :]
            for x in (q, k):
                a, b = x[..., :half].clone(), x[..., half:rot].clone()
                x[..., :half] = a * c - b * s
                x[..., half:rot] = a * s + b * c
        q_out.copy_(q.reshape(T, nh * d).to(q_out.dtype))
        if not cache.writes:
            return
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                continue
            pos = int(ctx.positions[t])
            page = int(table[r, pos // P])
            assert page >= 0
            cache.pages[page, 0, :, pos % P, :] = k[t].to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % P, :] = v[t].to(cache.pages.dtype)

    def paged_attention(self, q, out, ctx, cache, nh, nkv, d, scale, softcap, window, value_split=0, keep_first=0, sink=False):
        T = q.shape[0]
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        group = nh // nkv
        G = value_split
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                out[t] = 0
                continue
            pos = int(ctx.positions[t])
            lo = max(0, pos - window + 1) if window else 0
            js = list(range(0, min(keep_first, lo) if window else 0)) + list(range(lo, pos + 1))
            pages = [int(table[r, j // P]) for j in js]
            assert all(p >= 0 for p in pages), f"row {t} reads a page that was given back"
            slots = [j % P for j in js]
            K = cache.pages[pages, 0, :, slots, :].float()        # [n, nkv, d]
            V = cache.pages[pages, 1, :, slots, :].float()
            qt = q[t].float().view(nh // G if G else nh, d)
            for h in range(nh):
                if G:                          # result head h: query head qh over key head kh and value head vh
                    kh, vh = (h // group) // G, (h // group) % G
                    qh = kh * group + h % group
                else:
                    kh = vh = h // group
                    qh = h
                s = (K[:, kh] @ qt[qh]) * scale
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                if sink:                      # one more term, exp(0), in the denominator
                    p = torch.softmax(torch.cat([s, s.new_zeros(1)]), dim=0)[:-1]
                else:
                    p = torch.softmax(s, dim=0)
                out[t, h * d:(h + 1) * d] = (p @ V[:, vh]).to(out.dtype)

    # ---- short convolution, q|k|v preparation, state-space scan (restatements of what the kernels of the same names do) ----------------
    @staticmethod
    def _conv_inputs(proj, col0, in_bias, C, taps, state, ctx, req):
        """[taps - 1 + n, C]: the state of request `req` followed by its biased inputs of this step."""
        r0, n, slot = int(ctx.req_row_start[req]), int(ctx.req_n_rows[req]), int(ctx.req_state_slot[req])
        u = proj[r0:r0 + n, col0:col0 + C].float()
        if in_bias is not None:
            u = u + in_bias.float()[None, :]
        old = state[slot, :taps - 1].float() if (state is not None and taps > 1) else torch.zeros(0, C)
        return torch.cat([old, u], 0), r0, n, slot

    def short_conv(self, proj, col0, in_bias, weight, out_bias, act, state, out, ctx, commit_inline=False):
        C, taps = weight.shape
        for req in range(ctx.n_reqs):
            if int(ctx.req_n_rows[req]) <= 0:
                continue
            u, r0, n, _ = self._conv_inputs(proj, col0, in_bias, C, taps, state, ctx, req)
            y = torch.zeros(n, C)
            for j in range(taps):
                y += u[j:j + n] * weight[:, j].float()[None, :]
            if out_bias is not None:
                y = y + out_bias.float()[None, :]
            if act == "silu":
                y = y * torch.sigmoid(y)
            out[r0:r0 + n] = y
        return False                                   # the state is never moved on here: the caller runs the commit

    def short_conv_commit(self, proj, col0, in_bias, n_channels, taps, state, ctx, w_dtype=None):
        if taps <= 1:
            return
        for req in range(ctx.n_reqs):
            if int(ctx.req_n_rows[req]) <= 0:
                continue
            u, _, _, slot = self._conv_inputs(proj, col0, in_bias, n_channels, taps, state, ctx, req)
            state[slot, :taps - 1] = u[-(taps - 1):]

    def qkv_prepare(self, proj, col0, in_bias, conv_w, conv_state, q_norm, k_norm, eps, cos, sin, rot, interleaved,
                    nh, nkv, dk, dv, ctx, cache, q_out, commit_inline=False):
        T = q_out.shape[0]
        D = cache.pages.shape[-1]
        C = (nh + nkv) * dk + nkv * dv
        x = torch.zeros(T, C)
        if conv_w is not None:
            self.short_conv(proj, col0, in_bias, conv_w, None, None, conv_state, x, ctx)
        else:
            x = proj[:, col0:col0 + C].float() + (in_bias.float()[None, :] if in_bias is not None else 0.0)
        q = x[:, :nh * dk].reshape(T, nh, dk).clone()
        k = x[:, nh * dk:(nh + nkv) * dk].reshape(T, nkv, dk).clone()
        v = x[:, (nh + nkv) * dk:].reshape(T, nkv, dv)
        for y, w in ((q, q_norm), (k, k_norm)):
            if w is not None:
                y.copy_(y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w.float())
        if rot:
            c, s_ = cos[:, None, :], sin[:, None, :]
            for y in (q, k):
                if interleaved:
                    a, b = y[..., 0:rot:2].clone(), y[..., 1:rot:2].clone()
                    y[..., 0:rot:2] = a * c - b * s_
                    y[..., 1:rot:2] = b * c + a * s_
                else:
                    a, b = y[..., :rot // 2].clone(), y[..., rot // 2:rot].clone()
                    y[..., :rot // 2] = a * c - b * s_
                    y[..., rot // 2:rot] = a * s_ + b * c
        qp = torch.zeros(T, nh, D)
        qp[..., :dk] = q
        valid = (ctx.row_req[:T] >= 0)
        qp[~valid] = 0
        q_out.copy_(qp.reshape(T, nh * D).to(q_out.dtype))
        if not cache.writes:
            return False
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                continue
            pos = int(ctx.positions[t])
            page = int(table[r, pos // P])
            assert page >= 0
            cache.pages[page, :, :, pos % P, :] = 0
            cache.pages[page, 0, :, pos % P, :dk] = k[t].to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % P, :dv] = v[t].to(cache.pages.dtype)
        return False

    def head_gate(self, o, proj, gate_col0, nh, dv, D, out, ctx, out_col0=0, scale=1.0):
        T = out.shape[0]
        y = o.float().view(T, nh, D)[..., :dv]
        if proj is not None:
            y = y * torch.sigmoid(proj[:, gate_col0:gate_col0 + nh].float())[..., None]
        y = y * (ctx.row_req[:T] >= 0).float()[:, None, None] * scale
        out[:, out_col0:out_col0 + nh * dv] = y.reshape(T, nh * dv).to(out.dtype)

    def ssm_scan(self, xbc, proj, dt_col0, dt_bias, a_log, d_skip, state, y, heads, groups, P, N, ctx, writes=True):
        inner = heads * P
        A = -torch.exp(a_log.float())
        for req in range(ctx.n_reqs):
            n = int(ctx.req_n_rows[req])
            if n <= 0:
                continue
            r0, slot = int(ctx.req_row_start[req]), int(ctx.req_state_slot[req])
            S = state[slot].clone()                                   # [heads, P, N]
            for i in range(n):
                row = xbc[r0 + i]
                dt = torch.nn.functional.softplus(proj[r0 + i, dt_col0:dt_col0 + heads].float() + dt_bias.float(), threshold=20.0)
                for h in range(heads):
                    g = h // (heads // groups)
                    x = row[h * P:(h + 1) * P]
                    B = row[inner + g * N:inner + (g + 1) * N]
                    C = row[inner + groups * N + g * N:inner + groups * N + (g + 1) * N]
                    S[h] = torch.exp(A[h] * dt[h]) * S[h] + dt[h] * torch.outer(x, B)
                    y[r0 + i, h * P:(h + 1) * P] = S[h] @ C + d_skip[h].float() * x
            if writes:
                state[slot] = S

    def gated_group_norm(self, y, proj, z_col0, weight, eps, parts, out, ctx):
        T, inner = out.shape
        z = proj[:, z_col0:z_col0 + inner].float()
        v = (y * (z * torch.sigmoid(z))).view(T, parts, inner // parts)
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        v = v.reshape(T, inner) * weight.float()[None, :]
        v = torch.where((ctx.row_req[:T] >= 0)[:, None], v, torch.zeros_like(v))
        out.copy_(v.to(out.dtype))

    def add2_rmsnorm(self, a, b, x, *, next_weight=None, next_eps=0.0, next_plus_one=False, next_out=None):
        x.add_(a if b is None else a + b)
        if next_out is not None:
            self.rmsnorm(x, next_weight, next_eps, next_plus_one, next_out)

    # ---- gated delta rule, latent attention, layer scales, side inputs, mixtures of experts ---------------------------------
    def linear_cols(self, base, col0, weight, out):
        K = weight.shape[1]
        out.copy_((base[:, col0:col0 + K].float() @ weight.float().T).to(out.dtype))

    def delta_rule(self, qkv, q0, k0, v0, beta, beta0, decay, decay0, per_channel, dt_bias, a_log, state, out, heads, kv_heads,
                   dim, vdim, ctx, writes=True):
        rate = torch.exp(a_log.float())
        rep = heads // kv_heads
        for req in range(ctx.n_reqs):
            n = int(ctx.req_n_rows[req])
            if n <= 0:
                continue
            r0, slot = int(ctx.req_row_start[req]), int(ctx.req_state_slot[req])
            S = state[slot].clone()                                   # [heads, dim, vdim]
            for i in range(n):
                row = qkv[r0 + i].float()
                q = row[q0:q0 + kv_heads * dim].view(kv_heads, dim)
                k = row[k0:k0 + kv_heads * dim].view(kv_heads, dim)
                v = row[v0:v0 + heads * vdim].view(heads, vdim)
                q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
                k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
                b = torch.sigmoid(beta[r0 + i, beta0:beta0 + heads].float())
                if per_channel:
                    raw = decay[r0 + i, decay0:decay0 + heads * dim].float() + dt_bias.float()
                    g = torch.exp(-rate[:, None] * torch.nn.functional.softplus(raw, threshold=20.0).view(heads, dim))
                else:
                    raw = decay[r0 + i, decay0:decay0 + heads].float() + dt_bias.float()
                    g = torch.exp(-rate * torch.nn.functional.softplus(raw, threshold=20.0))[:, None].expand(heads, dim)
                for h in range(heads):
                    kh = h // rep
                    S[h] = S[h] * g[h][:, None]
                    u = b[h] * (v[h] - S[h].T @ k[kh])
                    S[h] = S[h] + torch.outer(k[kh], u)
                    out[r0 + i, h * vdim:(h + 1) * vdim] = S[h].T @ q[kh]
            if writes:
                state[slot] = S

    def head_norm_gate(self, o, weight, eps, gate, gate0, act, out, heads, vdim, out_col0=0, scale=1.0):
        T = out.shape[0]
        y = o[:T].float().view(T, heads, vdim)
        w = weight.float().view(heads, vdim)[None] if weight.numel() == heads * vdim else weight.float()[None, None, :]
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w
        z = gate[:T, gate0:gate0 + heads * vdim].float().view(T, heads, vdim)
        y = y * (z * torch.sigmoid(z) if act == "silu" else torch.sigmoid(z))
        out[:, out_col0:out_col0 + heads * vdim] = (torch.nan_to_num(y).reshape(T, heads * vdim) * scale).to(out.dtype)

    def latent_append(self, proj, c0, rank, weight, eps, ctx, cache):
        table = ctx.block_tables[cache.group]
        D = cache.pages.shape[-1]
        for t in range(proj.shape[0]):
            req = int(ctx.row_req[t])
            if req < 0:
                continue
            c = proj[t, c0:c0 + rank].float()
            c = c * torch.rsqrt(c.pow(2).mean() + eps) * weight.float()
            pos = int(ctx.positions[t])
            page = int(table[req, pos // cache.page_size])
            row = torch.zeros(D)
            row[:rank] = c
            cache.pages[page, 0, 0, pos % cache.page_size] = row.to(cache.pages.dtype)
            cache.pages[page, 1, 0, pos % cache.page_size] = row.to(cache.pages.dtype)

    def repeat_rows(self, a, b, parts, out_a, out_b):
        out_a.copy_(a.repeat_interleave(parts))
        out_b.copy_(b.repeat_interleave(parts))

    def head_linear(self, x, col0, weight, out):
        H, O, I = weight.shape
        T = out.shape[0]
        xs = x[:T, col0:col0 + H * I].float().view(T, H, I)
        out.copy_(torch.einsum("thi,hoi->tho", xs, weight.float()).reshape(T, H * O).to(out.dtype))

    def moe_route(self, logits, correction, groups, keep, top, scale, ids, weights, *, score="sigmoid", group_rank="best_two",
                  normalize=True):
        T, E = logits.shape
        z = torch.nan_to_num(logits.float())
        s = torch.softmax(z, dim=-1) if score == "softmax" else torch.sigmoid(z)
        choice = s + (correction.float()[None, :] if correction is not None else 0.0)
        if score == "sigmoid" and correction is None and groups == 1:
            choice = z                              # the same ranking, without the ties of a sigmoid that rounds to 1
        if groups > 1:
            per = E // groups
            g = choice.view(T, groups, per)
            score = g.topk(min(1 if group_rank == "best" else 2, per), dim=-1).values.sum(-1)
            best = score.topk(keep, dim=-1).indices
            ok = torch.zeros(T, groups, dtype=torch.bool).scatter_(1, best, True)
            choice = choice.masked_fill(~ok[:, :, None].expand(T, groups, per).reshape(T, E), float("-inf"))
        pick = choice.topk(top, dim=-1).indices
        w = s.gather(1, pick)
        ids.copy_(pick.to(torch.int32))
        weights.copy_((w / (w.sum(-1, keepdim=True) + 1e-20) if normalize else w) * scale)

    @staticmethod
    def _gnorm(x, weight, eps, groups):
        T, H = x.shape
        p = x.float().reshape(T, groups, H // groups)
        return (p * torch.rsqrt(p.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, H) * weight.float()

    def group_rmsnorm(self, x, weight, eps, groups, out, rows=None):
        src = x if rows is None else x[rows.long()]
        out.copy_(self._gnorm(src, weight, eps, groups).to(out.dtype))

    def add_group_rmsnorm(self, branch, weight, eps, groups, residual, *, shift=None, next_weight=None, next_eps=0.0,
                          next_out=None):
        if branch is not None:
            residual += self._gnorm(branch, weight, eps, groups)
        if shift is not None:
            residual += shift.float()[None, :]
        if next_out is not None:
            next_out.copy_(self._gnorm(residual, next_weight, next_eps, groups).to(next_out.dtype))

    def poly_norm(self, z, coef, eps, out):
        a, b, c, e = (float(v) for v in coef.float())
        z = z.float()

        def n(u):
            return u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps)

        out.copy_((a * n(z) + b * n(z * z) + c * n(z * z * z) + e).to(out.dtype))

    def rotate_norm_append(self, proj, col0, cos, sin, rot, magnitude, unit_norm, eps, nh, nkv, dk, dv, ctx, cache, q_out):
        T = q_out.shape[0]
        D = cache.pages.shape[-1]
        C = (nh + nkv) * dk + nkv * dv
        x = proj[:, col0:col0 + C].float()
        q = x[:, :nh * dk].reshape(T, nh, dk).clone()
        k = x[:, nh * dk:(nh + nkv) * dk].reshape(T, nkv, dk).clone()
        v = x[:, (nh + nkv) * dk:].reshape(T, nkv, dv)
        for y in (q, k):
            if rot:
                c, s_ = cos[:, None, :] * magnitude, sin[:, None, :] * magnitude
                a, b = y[..., :rot // 2].clone(), y[..., rot // 2:rot].clone()
                y[..., :rot // 2] = a * c - b * s_
                y[..., rot // 2:rot] = a * s_ + b * c
            if unit_norm:
                y.copy_(y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps))
        qp = torch.zeros(T, nh, D)
        qp[:, :, :dk] = q
        qp[ctx.row_req[:T] < 0] = 0
        q_out.copy_(qp.reshape(T, nh * D).to(q_out.dtype))
        if not cache.writes:
            return
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                continue
            pos = int(ctx.positions[t])
            page = int(table[r, pos // P])
            assert page >= 0
            cache.pages[page, :, :, pos % P, :] = 0
            cache.pages[page, 0, :, pos % P, :dk] = k[t].to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % P, :dv] = v[t].to(cache.pages.dtype)

    def head_mix_gate(self, o, mix, proj, gate_col0, nh, nkv, dv, D, out, ctx):
        T = out.shape[0]
        per = nh // nkv
        if mix is None:
            y = o.float().reshape(T, nh, D)[..., :dv].clone()
        else:
            wide = o.float().reshape(T, nh * nkv, D)[..., :dv]
            y = torch.zeros(T, nh, dv)
            for h in range(nh):
                for g in range(nh):
                    y[:, h] += mix[h, g].float() * wide[:, ((g // per) * nkv + h // per) * per + g % per]
        y = y.reshape(T, nh * dv)
        if proj is not None:
            y = y * torch.sigmoid(proj[:, gate_col0:gate_col0 + nh * dv].float())
        y[ctx.row_req[:T] < 0] = 0
        out.copy_(y.to(out.dtype))

    @staticmethod
    def _turn(y, cos, sin, rot, interleaved, magnitude):
        """y [T, heads, n]: the first `rot` elements of every head turned in place by the rows' angles."""
        if not rot:
            return
        c, s_ = cos[:, None, :] * magnitude, sin[:, None, :] * magnitude
        if interleaved:
            a, b = y[..., 0:rot:2].clone(), y[..., 1:rot:2].clone()
            y[..., 0:rot:2] = a * c - b * s_
            y[..., 1:rot:2] = b * c + a * s_
        else:
            a, b = y[..., :rot // 2].clone(), y[..., rot // 2:rot].clone()
            y[..., :rot // 2] = a * c - b * s_
            y[..., rot // 2:rot] = b * c + a * s_

    def rownorm_rope_append(self, proj, col0, bias, q_norm, k_norm, eps, cos, sin, rot, interleaved, magnitude, nh, nkv, dk, dv,
                            ctx, cache, q_out, v_mix=None, v_shared=None, v_mode=0):
        T = q_out.shape[0]
        D = cache.pages.shape[-1]
        C = (nh + nkv) * dk + nkv * dv
        x = proj[:T, col0:col0 + C].float()
        if bias is not None:
            x = x + bias.float()[None, :]
        q, k, v = x[:, :nh * dk].clone(), x[:, nh * dk:(nh + nkv) * dk].clone(), x[:, (nh + nkv) * dk:].clone()
        if q_norm is not None:
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm.float()
        if k_norm is not None:
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm.float()
        q, k, v = q.reshape(T, nh, dk), k.reshape(T, nkv, dk), v.reshape(T, nkv, dv)
        self._turn(q, cos, sin, rot, interleaved, magnitude)
        self._turn(k, cos, sin, rot, interleaved, magnitude)
        live = ctx.row_req[:T] >= 0
        if v_mode == 1 and cache.writes:
            v_shared[:T][live] = v.reshape(T, nkv * dv)[live]
        elif v_mode == 2:
            lam = float(v_mix.reshape(-1)[0])
            v = (1.0 - lam) * v + lam * v_shared[:T].float().view(T, nkv, dv)
        qp = torch.zeros(T, nh, D)
        qp[:, :, :dk] = q
        qp[~live] = 0
        q_out.copy_(qp.reshape(T, nh * D).to(q_out.dtype))
        if not cache.writes:
            return
        table = ctx.block_tables[cache.group]
        P = cache.page_size
        for t in range(T):
            r = int(ctx.row_req[t])
            if r < 0:
                continue
            pos = int(ctx.positions[t])
            page = int(table[r, pos // P])
            assert page >= 0
            cache.pages[page, :, :, pos % P, :] = 0
            cache.pages[page, 0, :, pos % P, :dk] = k[t].to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % P, :dv] = v[t].to(cache.pages.dtype)

    def cols_rmsnorm(self, x, c0, weight, eps, out):
        T, n = out.shape
        c = x[:T, c0:c0 + n].float()
        out.copy_((c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(out.dtype))

    def latent_rope_append(self, proj, c0, rank, rot, weight, eps, cos, sin, interleaved, magnitude, q, q0, n_heads, q_dim, ctx, cache):
        T = proj.shape[0]
        live = ctx.row_req[:T] >= 0
        heads = q[:T, q0:q0 + n_heads * (q_dim + rot)].view(T, n_heads, q_dim + rot)
        part = heads[..., q_dim:].clone()
        self._turn(part, cos[:T], sin[:T], rot, interleaved, magnitude)
        heads[..., q_dim:][live] = part[live]
        if not cache.writes:
            return
        table = ctx.block_tables[cache.group]
        D = cache.pages.shape[-1]
        kr = proj[:T, c0 + rank:c0 + rank + rot].float().reshape(T, 1, rot).clone()
        self._turn(kr, cos[:T], sin[:T], rot, interleaved, magnitude)
        for t in range(T):
            req = int(ctx.row_req[t])
            if req < 0:
                continue
            c = proj[t, c0:c0 + rank].float()
            c = c * torch.rsqrt(c.pow(2).mean() + eps) * weight.float()
            pos = int(ctx.positions[t])
            page = int(table[req, pos // cache.page_size])
            key, val = torch.zeros(D), torch.zeros(D)
            key[:rank] = val[:rank] = c
            key[rank:rank + rot] = kr[t, 0]
            cache.pages[page, 0, 0, pos % cache.page_size] = key.to(cache.pages.dtype)
            cache.pages[page, 1, 0, pos % cache.page_size] = val.to(cache.pages.dtype)

    def mlstm(self, proj, q0, k0, v0, i0, f0, bias_i, bias_f, cap, memory, norm_state, out, heads, dim, vdim, ctx, writes=True):
        H, d, dv = heads, dim, vdim
        for r in range(ctx.n_reqs):
            n, row0, slot = int(ctx.req_n_rows[r]), int(ctx.req_row_start[r]), int(ctx.req_state_slot[r])
            if n <= 0 or slot < 0:
                continue
            m_at = norm_state.shape[2] - 4                     # copies of n (one per 16 value columns), then m
            S, nn, m = memory[slot].float().clone(), norm_state[slot, :, :d].float().clone(), norm_state[slot, :, m_at].float().clone()
            for t in range(row0, row0 + n):
                x = proj[t].float()
                gi = cap * torch.tanh((x[i0:i0 + H] + bias_i.float()) / cap)
                gf = torch.nn.functional.logsigmoid(cap * torch.tanh((x[f0:f0 + H] + bias_f.float()) / cap))
                m_new = torch.maximum(gf + m, gi)
                keep, take = torch.exp(gf + m - m_new), torch.exp(gi - m_new)
                q = x[q0:q0 + H * d].view(H, d) * d ** -0.5
                k, v = x[k0:k0 + H * d].view(H, d), x[v0:v0 + H * dv].view(H, dv)
                S = keep[:, None, None] * S + take[:, None, None] * k[:, :, None] * v[:, None, :]
                nn = keep[:, None] * nn + take[:, None] * k
                m = m_new
                den = torch.maximum((nn * q).sum(-1).abs(), torch.exp(-m)) + 1e-6
                out[t] = (torch.einsum("hdv,hd->hv", S, q) / den[:, None]).reshape(H * dv)
            if writes:
                memory[slot] = S
                norm_state[slot, :, :m_at] = nn.repeat(1, m_at // d)
                norm_state[slot, :, m_at] = m

    def weighted_sum2(self, a, sa, b, sb, out):
        out.copy_(sa * a + sb * b)

    def convert(self, src, dst):
        dst.copy_(src.to(dst.dtype))

    def moe_plan(self, ids, n_experts, ctx):
        T, top = ids.shape
        flat = ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel())
        return {"pairs": T * top, "top": top, "sorted_pair": order.to(torch.int32), "inverse": inverse.to(torch.int32),
                "expert_of_sorted": flat[order]}

    def moe_linear(self, x, plan, weight, out, *, gather, gated=False, limit=0.0, activation="clamped_swish", row_scale=None):
        top = plan["top"]
        for r in range(plan["pairs"]):
            e = int(plan["expert_of_sorted"][r])
            row = x[int(plan["sorted_pair"][r]) // top] if gather else x[r]
            y = weight[e].float() @ row.float()
            if row_scale is not None:
                y = y * row_scale.reshape(-1)[int(plan["sorted_pair"][r])]
            if gated:
                N = y.shape[0] // 2
                y = y[:N] * torch.sigmoid(y[:N]) * y[N:] if activation == "silu" else self._clamped(y[:N], y[N:], limit)
            out[r] = y.to(out.dtype)

    def moe_combine(self, expert_out, plan, weights, shared, y):
        T, W = y.shape
        top = plan["top"]
        rows = expert_out[plan["inverse"].long()].view(T, top, W)
        acc = (rows * weights[:, :, None]).sum(1) if weights is not None else rows.sum(1)
        y.copy_(acc + (shared if shared is not None else 0.0))

    def scale_add_rmsnorm(self, a, scale, x, *, next_weight=None, next_eps=0.0, next_plus_one=False, next_out=None, copy_out=None):
        x.add_(a * scale.float()[None, :])
        if copy_out is not None:
            copy_out.copy_(x.to(copy_out.dtype))
        if next_out is not None:
            self.rmsnorm(x, next_weight, next_eps, next_plus_one, next_out)

    def side_gate(self, gate, tokens, table, col0, out):
        T, dim = out.shape
        e = table.float()[tokens[:T].long()][:, col0:col0 + dim]
        out.copy_((_act("gelu_tanh", gate.float()) * e).to(out.dtype))

    def activation(self, x, out, act):
        out.copy_(_act(act, x.float()).to(out.dtype))

    def linear_act(self, x, w_up, out, activation, ctx):
        out.copy_(_act(activation, x.float() @ w_up.float().T).to(out.dtype))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

    def sample(self, logits, states, out_ids, *, logit_rows=None, row_req=None, req_slot=None, whole_ranking=False,
               cand_ids=None, cand_vals=None, cand_lse=None):
        """The device sampler's stand-in: the plain sampler of tests/plain_sampler.py on each row, reading and updating
        the per-request state words as the kernels do."""
        import numpy as np
        import plain_sampler
        from kungfu_b200.sampling import RING, generator_state
        st_all = states.numpy()
        for i in range(logits.shape[0]):
            lr = i if logit_rows is None else int(logit_rows[i])
            rq = 0 if row_req is None else int(row_req[lr])
            if rq < 0:
                out_ids[i] = 0
                continue
            st = st_all[rq if req_slot is None else int(req_slot[rq])]
            f = st[2:6].view(np.float32)
            count = int(st[8])
            recent = [int(st[16 + j % RING]) for j in range(max(0, count - RING), count)]
            rng = plain_sampler.Rng(1)
            rng.state = generator_state(st)
            tok, _ = plain_sampler.sample(logits[i].float().numpy(), temperature=float(f[0]), top_k=int(st[6]), top_p=float(f[1]),
                                          min_p=float(f[2]), repeat_penalty=float(f[3]), repeat_window=int(st[7]),
                                          recent=recent, rng=rng)
            st[0:2] = np.array([rng.state & 0xFFFFFFFF, rng.state >> 32], dtype=np.uint32).view(np.int32)
            st[16 + count % RING] = tok
            st[8] = count + 1
            out_ids[i] = tok

    def topk_lse(self, logits, k, out_ids, out_vals, out_lse):
        V = logits.shape[1]
        # falling value, lower id first among equals
        order = torch.argsort(-logits.double() * 1.0, dim=-1, stable=True)[:, :k]
        out_ids.copy_(order.to(torch.int32))
        out_vals.copy_(torch.gather(logits, 1, order))
        out_lse.copy_(torch.logsumexp(logits.double(), dim=-1).float())
