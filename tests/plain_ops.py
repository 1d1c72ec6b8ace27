"""Plain references of the kernels, one function per kernel, on ordinary torch tensors.

Two uses.  The GPU tests compare each CUDA kernel with the function of the same name
here, at sizes other than the engine's.  And because `PlainOps` has the interface of
the product's kernel set, the CPU tests can drive the engine's host side (cache
manager, batch packing, step function, scheduler) through it without a GPU.  It is a
test double: the product never imports it and has no CPU path of its own.

Each function works in float32 (float64 where noted) whatever the storage dtype, and
loops over requests and tokens in the obvious way.
"""
from __future__ import annotations

import math

import torch


def _f(t):
    return t.to(torch.float32)


class PlainOps:
    name = "plain"

    # ---- embedding -------------------------------------------------------------------
    def embed(self, table, ids, out, scale=None):
        x = _f(table[ids.long()])
        out.copy_(x if scale is None else x * scale)

    # ---- residual add + RMSNorm ------------------------------------------------------
    def add_rmsnorm(self, resid, delta, weight, eps, out, rows=None, delta_scale=None, add=None):
        if delta is not None and delta_scale is not None:
            delta = _f(delta) * _f(delta_scale)
        if resid is None:
            x = _f(delta) if add is None else _f(delta) + _f(add)
        elif rows is None:
            if delta is not None:
                resid.add_(_f(delta))
            if add is not None:
                resid.add_(_f(add))
            x = resid
        else:
            x = resid[rows.long()]
            if delta is not None:
                x = x + _f(delta[rows.long()])
            if add is not None:
                x = x + _f(add)
        rms = (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt()
        out.copy_((x / rms * _f(weight)).to(out.dtype))

    # ---- matrix product --------------------------------------------------------------
    def linear(self, x, w, bias=None, out_dtype=None):
        y = _f(x) @ _f(w).t()
        if bias is not None:
            y = y + _f(bias)
        return y.to(out_dtype or x.dtype)

    def new_rows(self, n, width, dtype, device):
        return torch.empty((n, width), dtype=dtype, device=device)

    def linear_qk_norm_rope_write(self, x, w_qkv, num_heads, num_kv_heads, head_dim, q_weight,
                                  k_weight, eps, table, positions, slot_mapping, k_cache, v_cache,
                                  out_dtype=None):
        qkv = self.linear(x, w_qkv, out_dtype=out_dtype or x.dtype)
        self.qk_norm_rope_write(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps,
                                table, positions, slot_mapping, k_cache, v_cache)
        return qkv

    def add_bias(self, x, bias):
        x.copy_((_f(x) + _f(bias)).to(x.dtype))

    # ---- q/k norm + rotation + cache write -------------------------------------------
    def qk_norm_rope_write(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight,
                           eps, table, positions, slot_mapping, k_cache, v_cache):
        n = qkv.shape[0]
        hd, half = head_dim, head_dim // 2
        qd, kd = num_heads * hd, num_kv_heads * hd

        def norm_rotate(x, w):          # x: [n, heads, hd] float32
            if w is not None:
                x = x / (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt() * _f(w)
            if table is not None:
                cos = table[0][positions.long()].unsqueeze(1)
                sin = table[1][positions.long()].unsqueeze(1)
                a, b = x[..., :half], x[..., half:]
                x = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
            return x

        q = norm_rotate(_f(qkv[:, :qd]).reshape(n, num_heads, hd), q_weight)
        qkv[:, :qd] = q.reshape(n, qd).to(qkv.dtype).clone()
        if num_kv_heads:
            k = norm_rotate(_f(qkv[:, qd:qd + kd]).reshape(n, num_kv_heads, hd), k_weight)
            v = qkv[:, qd + kd:qd + 2 * kd].reshape(n, num_kv_heads, hd)
            kc = k_cache.view(-1, num_kv_heads, hd)
            vc = v_cache.view(-1, num_kv_heads, hd)
            for t in range(n):
                s = int(slot_mapping[t])
                if s >= 0:
                    kc[s] = k[t].to(kc.dtype)
                    vc[s] = v[t].to(vc.dtype)

    # ---- attention over the pages ----------------------------------------------------
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_cache, v_cache,
                        ctx, group, scale, window, out, sinks=None, v_head_dim=None):
        hd = head_dim
        vd = v_head_dim or head_dim
        G = num_heads // num_kv_heads
        ps = group.page_size
        q_start = ctx.q_start.tolist()
        ctx_lens = ctx.ctx_lens.tolist()
        for r in range(ctx.n_reqs):
            clen = ctx_lens[r]
            a, b = q_start[r], q_start[r + 1]
            if clen == 0:
                out[a:b] = 0
                continue
            table = group.block_table[r].tolist()
            for t in range(a, b):
                p = clen - (b - a) + (t - a)
                lo = 0 if window is None else max(0, p - window + 1)
                keys = list(range(lo, p + 1))
                idx = torch.tensor([table[j // ps] * ps + j % ps for j in keys])
                k = _f(k_cache.view(-1, num_kv_heads, hd)[idx])      # [keys, kv, hd]
                v = _f(v_cache.view(-1, num_kv_heads, vd)[idx])
                q = _f(qkv[t, :num_heads * hd]).reshape(num_heads, hd)
                for h in range(num_heads):
                    g = h // G
                    s = (k[:, g] @ q[h]) * scale
                    if sinks is not None:
                        s = torch.cat([s, _f(sinks[h:h + 1])])
                    pr = torch.softmax(s, dim=0)[:idx.shape[0]]
                    out[t, h * vd:(h + 1) * vd] = (pr @ v[:, g]).to(out.dtype)

    # ---- gated short convolution -----------------------------------------------------
    def short_conv(self, proj, filt, in_bias, conv_bias, state, ctx, out):
        hidden, taps = filt.shape
        q_start = ctx.q_start.tolist()
        slots = ctx.state_slot.tolist()
        start_pos = ctx.start_pos.tolist()
        p = _f(proj)
        if in_bias is not None:
            p = p + _f(in_bias)
        B, C, X = p[:, :hidden], p[:, hidden:2 * hidden], p[:, 2 * hidden:]
        bx = B * X
        for r in range(ctx.n_reqs):
            a, b = q_start[r], q_start[r + 1]
            slot = slots[r]
            if taps > 1 and slot >= 0 and start_pos[r] > 0:
                old = state[slot].clone()
            else:
                old = torch.zeros(taps - 1, hidden)
            rows = torch.cat([old, bx[a:b]], dim=0)
            n = b - a
            conv = torch.zeros(n, hidden)
            for k in range(taps):
                conv = conv + rows[k:k + n] * filt[:, k]
            if conv_bias is not None:
                conv = conv + _f(conv_bias)
            out[a:b] = (C[a:b] * conv).to(out.dtype)
            if taps > 1 and slot >= 0:
                state[slot] = rows[n:]

    # ---- SwiGLU activation -----------------------------------------------------------
    def swiglu(self, gate_up, out):
        f = out.shape[1]
        g, u = _f(gate_up[:, :f]), _f(gate_up[:, f:])
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    # ---- layer norm, alone or with the addition into the stream ------------------------
    def add_layernorm(self, resid, delta, weight, bias, eps, out, rows=None,
                      delta_weight=None, delta_bias=None, delta_eps=0.0):
        def ln(x, w, b, e):
            mu = x.mean(dim=-1, keepdim=True)
            var = (x - mu).pow(2).mean(dim=-1, keepdim=True)
            return (x - mu) / (var + e).sqrt() * _f(w) + _f(b)

        d = None if delta is None else _f(delta)
        if d is not None and delta_weight is not None:
            d = ln(d, delta_weight, delta_bias, delta_eps)
        if resid is None:
            x = d
        elif rows is None:
            if d is not None:
                resid.add_(d)
            x = resid
        else:
            x = resid[rows.long()]
            if d is not None:
                x = x + d[rows.long()]
        out.copy_(ln(x, weight, bias, eps).to(out.dtype))

    # ---- xIELU -----------------------------------------------------------------------
    def xielu(self, z, act, out):
        x = _f(z)
        sp = lambda a: torch.log1p(torch.exp(_f(a)))
        pos = sp(act[0]) * x * x + 0.5 * x
        neg = (0.5 + sp(act[1])) * (torch.expm1(torch.clamp(x, max=0.0)) - x) + 0.5 * x
        out.copy_(torch.where(x > 0, pos, neg).to(out.dtype))

    # ---- minGRU scan -----------------------------------------------------------------
    def mingru_scan(self, proj, bias, state, ctx, out):
        w = out.shape[1]
        q_start = ctx.q_start.tolist()
        slots = ctx.state_slot.tolist()
        p = _f(proj)
        for r in range(ctx.n_reqs):
            a, b = q_start[r], q_start[r + 1]
            if slots[r] < 0 or a == b:
                continue
            s = state[slots[r]].clone()
            for t in range(a, b):
                z = torch.sigmoid(p[t, :w] + _f(bias[:w]))
                u = p[t, w:2 * w] + _f(bias[w:])
                c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
                s = (1 - z) * s + z * c
                g = p[t, 2 * w:]
                out[t] = (s * g * torch.sigmoid(g)).to(out.dtype)
            state[slots[r]] = s

    # ---- partial rotation + cache write ------------------------------------------------
    def rope_partial_write(self, rows, num_heads, num_kv_heads, head_dim, v_head_dim, freq,
                           positions, slot_mapping, k_cache, v_cache):
        n = rows.shape[0]
        H, G, d, dv = num_heads, num_kv_heads, head_dim, v_head_dim

        def turn(x):                       # [n, heads, d] float32
            if freq is None:
                return x
            inv, dims = freq
            half = dims // 2
            a = positions.to(torch.float32)[:, None] * inv[None, :]
            cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
            u, v = x[..., :half], x[..., half:dims]
            return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)

        q = turn(_f(rows[:, :H * d]).reshape(n, H, d))
        rows[:, :H * d] = q.reshape(n, H * d).to(rows.dtype)
        if G:
            k = turn(_f(rows[:, H * d:(H + G) * d]).reshape(n, G, d))
            v = rows[:, (H + G) * d:(H + G) * d + G * dv].reshape(n, G, dv)
            kc, vc = k_cache.view(-1, G, d), v_cache.view(-1, G, dv)
            for t in range(n):
                s = int(slot_mapping[t])
                if s >= 0:
                    kc[s] = k[t].to(kc.dtype)
                    vc[s] = v[t].to(vc.dtype)

    # ---- attention with mixed heads over the pages ---------------------------------------
    def paged_attention_mixed(self, rows, gate_off, num_heads, num_kv_heads, head_dim, v_head_dim,
                              k_cache, v_cache, ctx, group, scale, window, chunk, head_mix, sinks,
                              out):
        H, G, d, dv = num_heads, num_kv_heads, head_dim, v_head_dim
        kv_of = torch.arange(H) // (H // G)
        ps = group.page_size
        q_start = ctx.q_start.tolist()
        ctx_lens = ctx.ctx_lens.tolist()
        for r in range(ctx.n_reqs):
            clen = ctx_lens[r]
            a, b = q_start[r], q_start[r + 1]
            if clen == 0:
                out[a:b] = 0
                continue
            table = group.block_table[r].tolist()
            for t in range(a, b):
                p = clen - (b - a) + (t - a)
                lo = 0 if window is None else max(0, p - window + 1)
                if chunk:
                    lo = max(lo, p // chunk * chunk)
                idx = torch.tensor([table[j // ps] * ps + j % ps for j in range(lo, p + 1)])
                k = _f(k_cache.view(-1, G, d)[idx])[:, kv_of]          # [keys, H, d]
                v = _f(v_cache.view(-1, G, dv)[idx])[:, kv_of]
                q = _f(rows[t, :H * d]).reshape(H, d)
                s = torch.einsum("hd,jhd->hj", q, k) * scale
                if head_mix is not None:
                    s = _f(head_mix) @ s
                if sinks is not None:
                    s = torch.cat([s, _f(sinks)[:, None]], dim=1)
                w = torch.softmax(s, dim=1)[:, :idx.shape[0]]
                o = torch.einsum("hj,jhd->hd", w, v).reshape(H * dv)
                if gate_off >= 0:
                    o = o * torch.sigmoid(_f(rows[t, gate_off:gate_off + H * dv]))
                out[t] = o.to(out.dtype)

    # ---- unit norm of q and k, query temperature, cache write ---------------------------
    def qk_unit_write(self, rows, num_heads, num_kv_heads, head_dim, v_head_dim, eps, q_temp,
                      positions, slot_mapping, k_cache, v_cache):
        n = rows.shape[0]
        H, G, d, dv = num_heads, num_kv_heads, head_dim, v_head_dim

        def unit(x):
            return x if eps is None else x / (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt()

        q = unit(_f(rows[:, :H * d]).reshape(n, H, d))
        if q_temp is not None:
            coef, every = q_temp
            steps = torch.div(positions.long() + 1, every, rounding_mode="floor") + 1
            q = q * (1.0 + coef * torch.log(steps.to(torch.float32)))[:, None, None]
        rows[:, :H * d] = q.reshape(n, H * d).to(rows.dtype).clone()
        if G:
            k = unit(_f(rows[:, H * d:(H + G) * d]).reshape(n, G, d))
            v = rows[:, (H + G) * d:(H + G) * d + G * dv].reshape(n, G, dv)
            kc, vc = k_cache.view(-1, G, d), v_cache.view(-1, G, dv)
            for t in range(n):
                s = int(slot_mapping[t])
                if s >= 0:
                    kc[s] = k[t].to(kc.dtype)
                    vc[s] = v[t].to(vc.dtype)

    # ---- latent rows: norm and cache write ----------------------------------------------
    def latent_norm_write(self, rows, offset, rank, weight, eps, slot_mapping, cache):
        c = _f(rows[:, offset:offset + rank])
        c = c / (c.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt() * _f(weight)
        pages = cache.view(-1, rank)
        for t in range(rows.shape[0]):
            s = int(slot_mapping[t])
            if s >= 0:
                pages[s] = c[t].to(pages.dtype)

    # ---- one small product per head -------------------------------------------------------
    def heads_product(self, rows, offset, heads, size, w, out, gate_rows=None, gate_off=-1):
        x = _f(rows[:, offset:offset + heads * size]).reshape(-1, heads, size)
        y = torch.einsum("nha,hab->nhb", x, _f(w)).reshape(out.shape)
        if gate_rows is not None:
            y = y * torch.sigmoid(_f(gate_rows[:, gate_off:gate_off + out.shape[1]]))
        out.copy_(y.to(out.dtype))

    def sigmoid_gate(self, x, rows, gate_off):
        g = torch.sigmoid(_f(rows[:, gate_off:gate_off + x.shape[1]]))
        x.copy_((_f(x) * g).to(x.dtype))

    # ---- mixture of experts ---------------------------------------------------------------
    def moe_select(self, logits, groups, keep, group_top, weight_eps, ids, weights,
                   score="sigmoid", renormalize=True, route_scale=1.0, choice_bias=None):
        n, E = logits.shape
        top = ids.shape[1]
        size = E // groups
        for t in range(n):
            s = torch.sigmoid(_f(logits[t])) if score == "sigmoid" else \
                torch.softmax(_f(logits[t]), dim=0)
            allowed = s.clone() if choice_bias is None else s + _f(choice_bias)
            if groups > 1:
                gs = allowed.reshape(groups, size).sort(dim=1, descending=True).values[:, :group_top].sum(1)
                kept = torch.sort(gs, descending=True, stable=True).indices[:keep].tolist()
                for g in range(groups):
                    if g not in kept:
                        allowed[g * size:(g + 1) * size] = -3.0e38
            chosen = torch.sort(allowed, descending=True, stable=True).indices[:top]
            ids[t] = chosen.to(torch.int32)
            w = s[chosen] / (s[chosen].sum() + weight_eps) if renormalize else s[chosen]
            weights[t] = w * route_scale

    def moe_route(self, x, router, groups, keep, group_top, weight_eps, ids, weights, **options):
        self.moe_select(_f(x) @ _f(router).t(), groups, keep, group_top, weight_eps, ids, weights,
                        **options)

    def moe_experts(self, x, ids, weights, gate_up, down, out, activation="swiglu", limit=0.0,
                    alpha=1.0, addend=None):
        n, top = ids.shape
        F = down.shape[2]
        y = torch.zeros((n, out.shape[1]), dtype=torch.float32)
        if addend is not None:
            y += _f(addend)
        for t in range(n):
            for k in range(top):
                e = int(ids[t, k])
                gu = _f(gate_up[e]) @ _f(x[t])               # gate and up rows alternate
                if activation == "relu2":                    # no gate: the up rows alone
                    act = gu.clamp(min=0).pow(2).to(x.dtype)
                elif activation == "glu_clamp":
                    g, u = gu[0::2].clamp(max=limit), gu[1::2].clamp(-limit, limit)
                    act = (g * torch.sigmoid(alpha * g) * (u + 1)).to(x.dtype)
                else:
                    act = (torch.nn.functional.silu(gu[0::2]) * gu[1::2]).to(x.dtype)
                y[t] += float(weights[t, k]) * (_f(down[e]) @ _f(act))
        out.copy_(y.to(out.dtype))

    def softcap(self, logits, cap):
        logits.copy_(cap * torch.tanh(logits / cap))

    # ---- relu squared; a sum of two mixers ---------------------------------------------
    def relu2(self, z, out):
        out.copy_(_f(z).clamp(min=0).pow(2).to(out.dtype))

    def weighted_sum(self, a, sa, b, sb, out):
        out.copy_((sa * _f(a) + sb * _f(b)).to(out.dtype))

    # ---- latent rows with a query latent and a turned key part ---------------------------
    @staticmethod
    def _turn(x, positions, freq):
        """x [n, ..., rot]: dimension i with i + rot/2 by the angle position * freq[i]."""
        half = x.shape[-1] // 2
        ang = positions.to(torch.float32)[:, None] * _f(freq)[None, :]
        shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
        cos, sin = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
        u, v = x[..., :half], x[..., half:]
        return torch.cat([u * cos - v * sin, v * cos + u * sin], dim=-1)

    def latent_prepare(self, rows, q_off, q_rank, q_weight, cq, kv_off, rank, rot, kv_weight, eps,
                       freq, positions, slot_mapping, cache):
        def norm(x, w):
            return x / (x.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt() * _f(w)
        if q_rank:
            cq.copy_(norm(_f(rows[:, q_off:q_off + q_rank]), q_weight).to(cq.dtype))
        c = norm(_f(rows[:, kv_off:kv_off + rank]), kv_weight)
        if rot:
            turned = self._turn(_f(rows[:, kv_off + rank:kv_off + rank + rot]), positions, freq)
            c = torch.cat([c, turned], dim=-1)
        pages = cache.view(-1, rank + rot)
        for t in range(rows.shape[0]):
            s = int(slot_mapping[t])
            if s >= 0:
                pages[s] = c[t].to(pages.dtype)

    def rope_heads(self, x, heads, size, off, rot, freq, positions):
        if not rot:
            return
        n = x.shape[0]
        v = x[:, :heads * size].reshape(n, heads, size)
        turned = self._turn(_f(v[..., off:off + rot]), positions, freq)
        v[..., off:off + rot] = turned.to(x.dtype)
        x[:, :heads * size] = v.reshape(n, heads * size)

    def head_gate(self, x, heads, size, rows, gate_off):
        g = torch.sigmoid(_f(rows[:, gate_off:gate_off + heads]))
        y = _f(x).reshape(-1, heads, size) * g[:, :, None]
        x.copy_(y.reshape(x.shape).to(x.dtype))

    # ---- matrix memory with exponential gates ----------------------------------------------
    def mlstm_record(self, heads, dim, vdim):
        return heads * (vdim + 1) * dim + heads

    def mlstm(self, rows, in_bias, forget_bias, norm_w, state, ctx, out, heads, dim, vdim, cap, eps):
        H, d, dv = heads, dim, vdim
        q_start = ctx.q_start.tolist()
        slots = ctx.state_slot.tolist()
        p = _f(rows)
        o_q, o_k, o_v = 0, H * d, 2 * H * d
        o_i = o_v + H * dv
        o_f, o_g = o_i + H, o_i + 2 * H
        for r in range(ctx.n_reqs):
            a, b = q_start[r], q_start[r + 1]
            if slots[r] < 0 or a == b:
                continue
            rec = state[slots[r]]
            C = rec[:H * (dv + 1) * d].reshape(H, dv + 1, d).clone()      # a column's rows side by side
            mx = rec[H * (dv + 1) * d:].clone()
            for t in range(a, b):
                li = cap * torch.tanh((p[t, o_i:o_i + H] + _f(in_bias)) / cap)
                lf = torch.nn.functional.logsigmoid(
                    cap * torch.tanh((p[t, o_f:o_f + H] + _f(forget_bias)) / cap))
                new = torch.maximum(lf + mx, li)
                keep, take = torch.exp(lf + mx - new), torch.exp(li - new)
                mx = new
                q = p[t, o_q:o_q + H * d].reshape(H, d) / math.sqrt(d)
                k = p[t, o_k:o_k + H * d].reshape(H, d)
                v = torch.cat([p[t, o_v:o_v + H * dv].reshape(H, dv), torch.ones(H, 1)], dim=1)
                C = keep[:, None, None] * C + take[:, None, None] * v[:, :, None] * k[:, None, :]
                read = torch.einsum("hcd,hd->hc", C, q)                   # [H, dv + 1]
                den = torch.maximum(read[:, dv].abs(), torch.exp(-mx)) + 1e-6
                o = read[:, :dv] / den[:, None]
                o = o / (o.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt()
                gate = torch.sigmoid(p[t, o_g:o_g + H * dv])
                out[t] = (o.reshape(H * dv) * _f(norm_w) * gate).to(out.dtype)
            rec[:H * (dv + 1) * d] = C.reshape(-1)
            rec[H * (dv + 1) * d:] = mx

    # ---- hyper-connections -----------------------------------------------------------
    def hyper_norm(self, src, dst, delta, mix, out_w, in_w, weight, eps, out, rows=None):
        x = src if src.dim() == 3 else None
        if x is None:
            S = dst.shape[1] if dst is not None else (in_w.shape[0] if in_w is not None else 1)
            x = src.unsqueeze(1).expand(-1, S, -1)
        x = x.clone()
        if delta is not None:
            x = torch.einsum("st,nsw->ntw", _f(mix), x) + _f(out_w)[None, :, None] * _f(delta)[:, None, :]
        if dst is not None:
            dst.copy_(x)
        if rows is not None:
            x = x[rows.long()]
        u = x.sum(1) if in_w is None else torch.einsum("t,ntw->nw", _f(in_w), x)
        rms = (u.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt()
        out.copy_((u / rms * _f(weight)).to(out.dtype))

    # ---- whole-projection q/k norm, pairwise rotation, value mixing, cache write -----
    def qkv_full_norm_rope_write(self, rows, bias, num_heads, num_kv_heads, head_dim, v_head_dim,
                                 q_weight, k_weight, eps, freq, rot_dims, positions, slot_mapping,
                                 q_out, k_cache, v_cache, v_first_in=None, v_first_out=None,
                                 lam=None):
        n = rows.shape[0]
        Q, K = num_heads * head_dim, num_kv_heads * head_dim
        x = _f(rows) if bias is None else _f(rows) + _f(bias)
        q, k, v = x[:, :Q], x[:, Q:Q + K], x[:, Q + K:]

        def norm(t, w):
            if w is None:
                return t
            return t / (t.pow(2).mean(dim=-1, keepdim=True) + eps).sqrt() * _f(w)

        def turn(t, heads):
            t = t.reshape(n, heads, head_dim).clone()
            if rot_dims:
                ang = positions.to(torch.float32)[:, None] * _f(freq)[None, :]
                c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
                a, b = t[..., 0:rot_dims:2].clone(), t[..., 1:rot_dims:2].clone()
                t[..., 0:rot_dims:2] = a * c - b * s
                t[..., 1:rot_dims:2] = b * c + a * s
            return t.reshape(n, heads * head_dim)

        q = turn(norm(q, q_weight), num_heads)
        k = turn(norm(k, k_weight), num_kv_heads)
        if v_first_out is not None:
            v_first_out.copy_(v)
        if v_first_in is not None:
            v = (1 - _f(lam)) * v + _f(lam) * _f(v_first_in)
        q_out.copy_(q.to(q_out.dtype))
        kc = k_cache.view(-1, K)
        vc = v_cache.view(-1, v.shape[1])
        for t in range(n):
            slot = int(slot_mapping[t])
            if slot >= 0:
                kc[slot] = k[t].to(kc.dtype)
                vc[slot] = v[t].to(vc.dtype)

    # ---- gated delta rule ------------------------------------------------------------
    def gated_delta_record(self, heads, kv_heads, dim, vdim, taps):
        return (taps - 1) * (2 * kv_heads * dim + heads * vdim) + heads * dim * vdim

    def gated_delta(self, proj, lowrank, filt, a_log, dt_bias, norm_w, state, ctx, out, heads,
                    kv_heads, dim, vdim, taps, unit_eps, eps):
        H, G, d, dv = heads, kv_heads, dim, vdim
        C = 2 * G * d + H * dv
        q_start = ctx.q_start.tolist()
        slots = ctx.state_slot.tolist()
        p, low = _f(proj), _f(lowrank)
        for r in range(ctx.n_reqs):
            a, b = q_start[r], q_start[r + 1]
            if slots[r] < 0 or a == b:
                continue
            rec = state[slots[r]]
            old = rec[:(taps - 1) * C].reshape(taps - 1, C).clone()
            S = rec[(taps - 1) * C:].reshape(H, d, dv).clone()
            rows = torch.cat([old, p[a:b, :C]], dim=0)
            n = b - a
            conv = torch.zeros(n, C)
            for j in range(taps):
                conv = conv + rows[j:j + n] * _f(filt)[:, j]
            act = conv * torch.sigmoid(conv)
            for i in range(n):
                t = a + i
                q = act[i, :G * d].reshape(G, d)
                k = act[i, G * d:2 * G * d].reshape(G, d)
                v = act[i, 2 * G * d:].reshape(H, dv)
                q = q / (q.pow(2).sum(-1, keepdim=True) + unit_eps).sqrt() / math.sqrt(d)
                k = k / (k.pow(2).sum(-1, keepdim=True) + unit_eps).sqrt()
                beta = torch.sigmoid(p[t, C:C + H])
                decay = torch.exp(-torch.exp(_f(a_log))[:, None] * torch.nn.functional.softplus(
                    low[t, :H * d] + _f(dt_bias)).reshape(H, d))
                gate = torch.sigmoid(low[t, H * d:H * d + H * dv]).reshape(H, dv)
                for h in range(H):
                    kh, qh = k[h // (H // G)], q[h // (H // G)]
                    S[h] = decay[h][:, None] * S[h]
                    u = beta[h] * (v[h] - S[h].t() @ kh)
                    S[h] = S[h] + torch.outer(kh, u)
                    o = S[h].t() @ qh
                    o = o / (o.pow(2).mean() + eps).sqrt() * _f(norm_w) * gate[h]
                    out[t, h * dv:(h + 1) * dv] = o.to(out.dtype)
            rec[:(taps - 1) * C] = rows[n:].reshape(-1)
            rec[(taps - 1) * C:] = S.reshape(-1)

    # ---- clamped gated activation ----------------------------------------------------
    def glu_clamp(self, gate_up, bias, out, limit, alpha):
        f = out.shape[1]
        x = _f(gate_up) if bias is None else _f(gate_up) + _f(bias)
        g, u = x[:, :f].clamp(max=limit), x[:, f:].clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(alpha * g) * (u + 1)).to(out.dtype))

    # ---- sampling --------------------------------------------------------------------
    def argmax(self, logits):
        out = torch.zeros(logits.shape[0], dtype=torch.int32)
        for m in range(logits.shape[0]):
            best, best_v = 0, float("-inf")
            for i, v in enumerate(logits[m].tolist()):
                if v > best_v:
                    best, best_v = i, v
            out[m] = best
        return out

    def sample(self, logits, temperature, top_p, seed, counter):
        out = torch.zeros(logits.shape[0], dtype=torch.int32)
        for m in range(logits.shape[0]):
            out[m] = sample_row(logits[m], float(temperature[m]), float(top_p[m]),
                                int(seed[m]), int(counter[m]))
        return out


# ---- the sampler's definition, restated --------------------------------------------

MASK64 = (1 << 64) - 1


def uniform(seed: int, counter: int) -> float:
    """The draw for (seed, counter): a splitmix64 finaliser over seed + (counter + 1) *
    the golden-ratio increment; the top 24 bits make a float in [0, 1)."""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample_row(logits, temperature: float, top_p: float, seed: int, counter: int) -> int:
    """Temperature and nucleus sampling of one row, in float64.

    temperature <= 0: first maximum.  Else p = softmax(logits / T); the nucleus is the
    set {p_i >= tau} for the largest tau whose set has mass >= top_p (ties with the last
    kept token are kept); the token is the first, in index order, whose cumulative
    kept mass reaches u * kept mass.
    """
    if temperature <= 0:
        return int(PlainOps().argmax(logits.unsqueeze(0))[0])
    z = logits.double() / temperature
    p = torch.exp(z - z.max())
    if top_p < 1.0:
        total = p.sum()
        order = torch.argsort(p, descending=True, stable=True)
        cum = torch.cumsum(p[order], 0)
        hit = (cum >= top_p * total).nonzero()
        cut = int(hit[0]) if len(hit) else len(p) - 1
        p = torch.where(p >= p[order[cut]], p, torch.zeros_like(p))
    r = uniform(seed, counter) * float(p.sum())
    cum = torch.cumsum(p, 0)
    hit = ((cum >= r) & (p > 0)).nonzero()
    return int(hit[0]) if len(hit) else int((p > 0).nonzero()[-1])
