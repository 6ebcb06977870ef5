"""Plain PyTorch references of the device operations, one per kernel, with the
signatures of ``tiny_inference_server_b200.kernels.ops``.

They serve two purposes: the GPU tests compare each CUDA kernel alone with its reference
here (at sizes other than the engine's), and the CPU tests put them in place of the
kernels (``install``) so that the cache manager, the step function, the scheduler and
trace replay can be checked where there is no GPU.  They are slow and obvious on
purpose; nothing of the product imports this file.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def _row_factor(scaled):
    """The norm's factor of each row from the partial sums of squares: "l2_eps": sqrt(width) / (||row|| + eps);
    "mean_eps": 1 / sqrt(mean of squares + eps)."""
    d = scaled.rows.shape[1]
    s = scaled.parts.sum(-1, keepdim=True)
    if scaled.kind == "mean_eps":
        return 1.0 / torch.sqrt(s / d + scaled.eps)
    return math.sqrt(d) / (s.sqrt() + scaled.eps)


def scaled_rows_dense(scaled):
    return (scaled.rows.to(torch.float32) * _row_factor(scaled)).to(scaled.rows.dtype)


def gemm(a, w, out=None, sink=None):
    """``a`` may be ``ops.ScaledRows`` (the product is multiplied by each row's factor afterwards); with a
    ``sink`` of matching shape and few bfloat16 rows the product is added to the stream there and the
    stream times the next norm's weight comes back with partial sums of squares by strip of 64 columns."""
    from tiny_inference_server_b200.kernels import ops
    factor = None
    if isinstance(a, ops.ScaledRows):
        factor, a = _row_factor(a), a.rows
    r = a.to(torch.float32) @ w.to(torch.float32)
    if factor is not None:
        r = r * factor
    if (sink is not None and out is None and a.dtype == torch.bfloat16 and a.shape[0] <= ops.SKINNY_MAX_ROWS
            and tuple(sink.values.shape) == tuple(r.shape)):
        sink.values += r
        n, d = r.shape
        strips = -(-d // 64)
        sq = torch.zeros((n, strips * 64), dtype=torch.float32)
        sq[:, :d] = sink.values.pow(2)
        return ops.ScaledRows((sink.values * sink.weight).to(a.dtype), sq.reshape(n, strips, 64).sum(-1), sink.eps, sink.norm,
                              sink.kind)
    r = r.to(a.dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def gemm_f32_out(a, w):
    return a.to(torch.float32) @ w.to(torch.float32)


def embed_rows(table, tokens, out, scale=1.0):
    out.copy_(table[tokens.long()].to(torch.float32) * scale)
    return out


def _norm_factor(x, eps, kind):
    d = x.shape[-1]
    if kind == "mean_eps":
        return 1.0 / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return math.sqrt(d) / (x.pow(2).sum(-1, keepdim=True).sqrt() + eps)


def add_rmsnorm(residual, delta, scale, eps, out, kind="l2_eps", delta_norm=None):
    if delta is not None:
        d32 = delta.to(torch.float32)
        if delta_norm is not None:
            dw, deps, dkind = delta_norm
            d32 = d32 * _norm_factor(d32, deps, dkind) * dw
        residual += d32
    if out is None:
        return None
    d = residual.shape[-1]
    if kind == "mean_eps":
        out.copy_((residual / torch.sqrt(residual.pow(2).mean(-1, keepdim=True) + eps) * scale).to(out.dtype))
        return out
    norm = residual.pow(2).sum(-1, keepdim=True).sqrt()
    out.copy_((residual * math.sqrt(d) / (norm + eps) * scale).to(out.dtype))
    return out


def glu_clamped(gu, gate_bias, up_bias, limit, alpha, shift, out, hidden):
    g = gu[:, :hidden].to(torch.float32)
    u = gu[:, hidden:2 * hidden].to(torch.float32)
    if gate_bias is not None:
        g = g + gate_bias
    if up_bias is not None:
        u = u + up_bias
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    out[:, :hidden] = (g * torch.sigmoid(alpha * g) * (u + shift)).to(out.dtype)
    out[:, hidden:] = 0
    if out.shape[1] > hidden:
        out[:, hidden] = 1
    return out


def scale_f32(x, scale):
    x *= scale
    return x


def softcap_f32(x, cap):
    x.copy_(cap * torch.tanh(x / cap))
    return x


def activation(x, out, kind):
    z = x.to(torch.float32)
    if kind == "relu2":
        y = torch.clamp(z, min=0.0) ** 2
    elif kind == "gelu_tanh":
        y = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
    else:
        y = z * torch.sigmoid(z)
    out.copy_(y.to(out.dtype))
    return out


def gemm_act(a, w, kind):
    h = gemm(a, w)
    return activation(h, h, kind)


def _segments(row_slot):
    """[(first row, rows, slot)] of the requests of a step (rows of a request are consecutive)."""
    segs = []
    slots = [int(s) for s in row_slot]
    for r, s in enumerate(slots):
        if s < 0:
            continue
        if segs and segs[-1][2] == s and segs[-1][0] + segs[-1][1] == r:
            segs[-1] = (segs[-1][0], segs[-1][1] + 1, s)
        else:
            segs.append((r, 1, s))
    return segs


def causal_conv(x, weight, state, out, row_slot, row_last, residual=False, silu=False, bias=None):
    taps, c = weight.shape
    hist = taps - 1
    for r0, rows, slot in _segments(row_slot):
        assert int(row_last[r0]) == r0 + rows - 1
        old = state[slot, :hist * c].reshape(hist, c).to(torch.float32)
        seq = torch.cat([old, x[r0:r0 + rows].to(torch.float32)], dim=0)          # positions -hist .. rows-1
        y = torch.zeros((rows, c), dtype=torch.float32)
        for j in range(taps):
            y += weight[j] * seq[j:j + rows]
        if bias is not None:
            y += bias
        if residual:
            y += seq[hist:]
        if silu:
            y = y * torch.sigmoid(y)
        out[r0:r0 + rows] = y.to(out.dtype)
        if hist:
            state[slot, :hist * c] = seq[rows:].reshape(-1)
    return out


def norm_mix_store(qkv, nq, nk, nv, q_weight, k_weight, eps, v_other, mix, k_pages, v_pages, block_table, positions,
                   row_slot, page_size, fault):
    kv_heads = k_pages.shape[1]
    for r in range(qkv.shape[0]):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        row = qkv[r].to(torch.float32)
        q, k, v = row[:nq], row[nq:nq + nk], row[nq + nk:nq + nk + nv]
        if q_weight is not None:
            qkv[r, :nq] = (q / torch.sqrt(q.pow(2).mean() + eps) * q_weight).to(qkv.dtype)
        if k_weight is not None:
            k = k / torch.sqrt(k.pow(2).mean() + eps) * k_weight
        if v_other is not None:
            lam = float(mix[0])
            v = (1.0 - lam) * v + lam * v_other[r].to(torch.float32)
        page = int(block_table[slot, pos // page_size])
        if page < 0 or page >= k_pages.shape[0]:
            fault[0] = 3
            continue
        k_pages[page, :, pos % page_size, :] = k.view(kv_heads, -1).to(k_pages.dtype)
        v_pages[page, :, pos % page_size, :] = v.view(kv_heads, -1).to(v_pages.dtype)


def window_attention(q, gate, out, k_pages, v_pages, block_table, positions, row_slot, num_heads, page_size, window,
                     scale, bias_slope, bias_rate, fault, step=None, sink=None, gate_per_head=False):
    kv_heads, k_dim, v_dim = k_pages.shape[1], k_pages.shape[3], v_pages.shape[3]
    g = num_heads // kv_heads
    for r in range(q.shape[0]):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        lo = max(0, pos - window + 1) if window else 0
        idx = torch.arange(lo, pos + 1)
        pages = block_table[slot, idx // page_size].long()
        k = k_pages[pages, :, idx % page_size, :].to(torch.float32).repeat_interleave(g, dim=1)     # (L, H, k_dim)
        v = v_pages[pages, :, idx % page_size, :].to(torch.float32).repeat_interleave(g, dim=1)
        qq = q[r].to(torch.float32).view(num_heads, k_dim)
        s = torch.einsum("hd,khd->hk", qq, k) * scale
        if bias_slope is not None:
            s = s - bias_slope[:, None] * torch.log(1.0 + bias_rate[:, None] * (pos - idx).to(torch.float32)[None, :])
        if sink is not None:               # one more term in the denominator, without a value
            s = torch.cat([s, sink.to(torch.float32)[:, None]], dim=-1)
        w = torch.softmax(s, dim=-1)[:, :idx.shape[0]]
        o = torch.einsum("hk,khd->hd", w, v)
        if gate is not None and gate_per_head:
            o = o * torch.sigmoid(gate[r, :num_heads].to(torch.float32))[:, None]
        o = o.reshape(-1)
        if gate is not None and not gate_per_head:
            o = o * torch.sigmoid(gate[r].to(torch.float32))
        out[r] = o.to(out.dtype)
    return out


def delta_rule(qkv, beta, decay_in, gate, a_log, dt_bias, norm_weight, eps, unit_eps, q_scale, state, out, row_slot,
               row_last, num_heads, qk_heads, k_dim, v_dim, requests=None, segments=None, decay_per_head=False,
               gate_act="sigmoid"):
    H, G = num_heads, qk_heads
    nq = G * k_dim
    rate = torch.exp(a_log.to(torch.float32))[:, None]
    for r0, rows, slot in _segments(row_slot):
        S = state[slot, :H * k_dim * v_dim].reshape(H, k_dim, v_dim).to(torch.float32).clone()
        for r in range(r0, r0 + rows):
            row = qkv[r].to(torch.float32)
            q = row[:nq].view(G, k_dim)
            k = row[nq:2 * nq].view(G, k_dim)
            v = row[2 * nq:2 * nq + H * v_dim].view(H, v_dim)
            q = (q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * q_scale).repeat_interleave(H // G, dim=0)
            k = (k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(H // G, dim=0)
            b = torch.sigmoid(beta[r].to(torch.float32))[:, None]
            if decay_per_head:
                a = (decay_in[r].to(torch.float32) + dt_bias)[:, None]
            else:
                a = decay_in[r].to(torch.float32).view(H, k_dim) + dt_bias.view(H, k_dim)
            S = torch.exp(-rate * torch.nn.functional.softplus(a))[:, :, None] * S
            u = b * (v - torch.einsum("hdv,hd->hv", S, k))
            S = S + k[:, :, None] * u[:, None, :]
            o = torch.einsum("hdv,hd->hv", S, q)
            o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_weight
            if gate is not None:
                gv = gate[r].to(torch.float32).view(H, v_dim)
                o = o * (torch.sigmoid(gv) if gate_act == "sigmoid" else gv * torch.sigmoid(gv))
            out[r] = o.reshape(-1).to(out.dtype)
        state[slot, :H * k_dim * v_dim] = S.reshape(-1)
    return out


def linear_attention(qkv, gate, decay, norm_weight, eps, state, out, row_slot, row_last, num_heads, k_dim, v_dim,
                     requests=None, segments=None):
    H = num_heads
    nq = H * k_dim
    act = torch.nn.functional.silu
    for r0, rows, slot in _segments(row_slot):
        S = state[slot, :H * k_dim * v_dim].reshape(H, k_dim, v_dim).to(torch.float32).clone()
        for r in range(r0, r0 + rows):
            row = qkv[r].to(torch.float32)
            q, k = act(row[:nq]).view(H, k_dim), act(row[nq:2 * nq]).view(H, k_dim)
            v = act(row[2 * nq:2 * nq + H * v_dim]).view(H, v_dim)
            S = decay.to(torch.float32)[:, None, None] * S + k[:, :, None] * v[:, None, :]
            o = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
            o = o / torch.sqrt(o.pow(2).mean() + eps) * norm_weight
            if gate is not None:
                o = o * torch.sigmoid(gate[r].to(torch.float32))
            out[r] = o.to(out.dtype)
        state[slot, :H * k_dim * v_dim] = S.reshape(-1)
    return out


def forget_gate_recurrence(qv, f_in, lower, f_bias, norm_weight, eps, state, out, row_slot, row_last, num_heads, k_dim,
                           v_dim, requests=None, segments=None):
    H = num_heads
    nq = H * k_dim
    low = lower.to(torch.float32).view(H, k_dim)
    for r0, rows, slot in _segments(row_slot):
        S = state[slot, :H * k_dim * v_dim].reshape(H, k_dim, v_dim).to(torch.float32).clone()
        for r in range(r0, r0 + rows):
            row = qv[r].to(torch.float32)
            q = torch.nn.functional.silu(row[:nq]).view(H, k_dim)
            v = row[nq:nq + H * v_dim].view(H, v_dim)
            f = low + (1.0 - low) * torch.sigmoid(f_in[r].to(torch.float32).view(H, k_dim) + f_bias.view(H, k_dim))
            S = f[:, :, None] * S + (1.0 - f)[:, :, None] * v[:, None, :]
            o = torch.einsum("hdv,hd->hv", S, q)
            o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_weight
            out[r] = o.reshape(-1).to(out.dtype)
        state[slot, :H * k_dim * v_dim] = S.reshape(-1)
    return out


def head_norm_store(qkv, num_heads, kv_heads, maps, dim, v_dim, bias, q_weight, k_weight, eps, temp_coef, temp_every,
                    q_out, k_pages, v_pages, block_table, positions, row_slot, page_size, fault):
    H, G, M = num_heads, kv_heads, maps
    nq, nk, nv = H * M * dim, G * M * dim, G * v_dim
    for r in range(qkv.shape[0]):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        row = qkv[r, :nq + nk + nv].to(torch.float32)
        if bias is not None:
            row = row + bias
        q, k, v = row[:nq].view(H, M, dim), row[nq:nq + nk].view(G, M, dim), row[nq + nk:].view(G, v_dim)
        if q_weight is not None:
            q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight
        if k_weight is not None:
            k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight
        if temp_every > 0:
            q = q * (1.0 + temp_coef * math.log((pos + 1) // temp_every + 1.0))
        wide = torch.zeros((H, M, M, dim), dtype=torch.float32)
        for m in range(M):
            wide[:, m, m] = q[:, m]
        q_out[r] = wide.reshape(-1).to(q_out.dtype)
        page = int(block_table[slot, pos // page_size])
        if page < 0 or page >= k_pages.shape[0]:
            fault[0] = 7
            continue
        k_pages[page, :, pos % page_size, :] = k.reshape(G, M * dim).to(k_pages.dtype)
        v_pages[page, :, pos % page_size, :] = v.to(v_pages.dtype)


def diff_combine(a, lam, eps, out_scale, out, num_heads, v_dim, row_slot=None):
    x = a.to(torch.float32).view(a.shape[0], num_heads, 2, v_dim)
    o = x[:, :, 0] - lam * x[:, :, 1]
    o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_scale
    out.copy_(o.reshape(a.shape[0], -1).to(out.dtype))
    return out


def latent_prepare(proj, dkv_at, num_heads, flat_dim, rot_dim, rank, c_weight, eps, cos, sin, q_out, k_pages, block_table,
                   positions, row_slot, page_size, fault):
    half = cos.shape[1] if cos is not None else 0
    qd, row_w = flat_dim + rot_dim, rank + rot_dim

    def turn(x, c, s):
        if half == 0:
            return x
        a, b = x[..., :half], x[..., half:2 * half]
        return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], dim=-1)

    for r in range(proj.shape[0]):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        row = proj[r].to(torch.float32)
        c, s = (cos[pos], sin[pos]) if cos is not None else (None, None)
        q_rot = row[:num_heads * qd].view(num_heads, qd)[:, flat_dim:]
        q_out[r].view(num_heads, row_w)[:, rank:] = turn(q_rot, c, s).to(q_out.dtype)
        low = row[dkv_at:dkv_at + row_w]
        latent = low[:rank] / torch.sqrt(low[:rank].pow(2).mean() + eps) * c_weight
        page = int(block_table[slot, pos // page_size])
        if page < 0 or page >= k_pages.shape[0]:
            fault[0] = 6
            continue
        k_pages[page, 0, pos % page_size, :] = torch.cat([latent, turn(low[rank:], c, s)]).to(k_pages.dtype)


def gemm_heads(a, w, out):
    out.copy_(torch.einsum("nhk,hkj->nhj", a.to(torch.float32), w.to(torch.float32)).to(out.dtype))
    return out


def moe_route(x, w_router, correction, w_shared_gate, groups, keep, top, weight_eps=1e-20, scores="sigmoid"):
    xf = x.to(torch.float32)
    s = xf @ w_router.t() if scores == "softmax_chosen" else torch.sigmoid(xf @ w_router.t())
    n, experts = s.shape
    pick = s + correction if correction is not None else s.clone()
    if groups:
        per = pick.view(n, groups, experts // groups)
        strength = per.topk(min(2, experts // groups), dim=-1).values.sum(-1)
        best = strength.topk(keep, dim=-1).indices
        ok = torch.zeros((n, groups), dtype=torch.bool).scatter_(1, best, True)
        pick = per.masked_fill(~ok[:, :, None], float("-inf")).reshape(n, experts)
    chosen = pick.topk(top, dim=-1).indices
    w = s.gather(1, chosen)
    w = torch.softmax(w, dim=-1) if scores == "softmax_chosen" else w / (w.sum(-1, keepdim=True) + weight_eps)
    shared = torch.sigmoid(xf @ w_shared_gate) if w_shared_gate is not None else None
    return chosen.to(torch.int32), w, shared


def _act(z, kind):
    if kind == "relu2":
        return torch.clamp(z, min=0.0) ** 2
    if kind == "gelu_tanh":
        return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    return z * torch.sigmoid(z)


def moe_gate_up(x, chosen, w_gate_up, act=None):
    n, top = chosen.shape
    xf = x.to(torch.float32)
    if act is not None:
        u = torch.einsum("ntfd,nd->ntf", w_gate_up.to(torch.float32)[chosen.long()], xf)
        return _act(u, act).reshape(n * top, -1).to(x.dtype)
    w = w_gate_up.to(torch.float32)[chosen.long()]                      # (n, top, 2, F, d)
    g = torch.einsum("ntfd,nd->ntf", w[:, :, 0], xf)
    u = torch.einsum("ntfd,nd->ntf", w[:, :, 1], xf)
    return (g * torch.sigmoid(g) * u).reshape(n * top, -1).to(x.dtype)


def moe_experts(x, chosen, weights, w_gate_up, w_down, shared, shared_gate, act=None):
    return moe_down(moe_gate_up(x, chosen, w_gate_up, act), chosen, weights, w_down, shared, shared_gate)


def gated_linear_attention(qkv, a_in, power, a_bias, gate, norm_weight, eps, q_scale, state, out, row_slot, row_last,
                           num_heads, k_dim, v_dim, requests=None, segments=None, gate_act="silu"):
    H = num_heads
    nq = H * k_dim
    for r0, rows, slot in _segments(row_slot):
        S = state[slot, :H * k_dim * v_dim].reshape(H, k_dim, v_dim).to(torch.float32).clone()
        for r in range(r0, r0 + rows):
            row = qkv[r].to(torch.float32)
            q = row[:nq].view(H, k_dim) * q_scale
            k = row[nq:2 * nq].view(H, k_dim)
            v = row[2 * nq:2 * nq + H * v_dim].view(H, v_dim)
            z = a_in[r].to(torch.float32).view(H, k_dim) + a_bias.view(H, k_dim)
            alpha = torch.exp(torch.nn.functional.logsigmoid(z) * power.view(H, 1))
            S = alpha[:, :, None] * S + k[:, :, None] * v[:, None, :]
            o = torch.einsum("hdv,hd->hv", S, q)
            o = (o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_weight).reshape(-1)
            if gate is not None:
                g = gate[r].to(torch.float32)
                o = o * (g * torch.sigmoid(g) if gate_act == "silu" else torch.sigmoid(g))
            out[r] = o.to(out.dtype)
        state[slot, :H * k_dim * v_dim] = S.reshape(-1)
    return out


def state_space_scan(cbx, dt_in, a_log, dt_bias, state, row_slot, row_last, num_heads, groups, state_dim, v_dim,
                     requests=None, segments=None):
    H, G, N = num_heads, groups, state_dim
    raw = torch.zeros((cbx.shape[0], H * v_dim), dtype=torch.float32)
    head_group = torch.arange(H) // (H // G)
    for r0, rows, slot in _segments(row_slot):
        S = state[slot, :H * N * v_dim].reshape(H, N, v_dim).to(torch.float32).clone()
        for r in range(r0, r0 + rows):
            row = cbx[r].to(torch.float32)
            C = row[:G * N].view(G, N)[head_group]
            B = row[G * N:2 * G * N].view(G, N)[head_group]
            x = row[2 * G * N:2 * G * N + H * v_dim].view(H, v_dim)
            dt = torch.nn.functional.softplus(dt_in[r].to(torch.float32)[:H] + dt_bias)
            S = torch.exp(-torch.exp(a_log) * dt)[:, None, None] * S + B[:, :, None] * (dt[:, None] * x)[:, None, :]
            raw[r] = torch.einsum("hnv,hn->hv", S, C).reshape(-1)
        state[slot, :H * N * v_dim] = S.reshape(-1)
    return raw


def skip_gate_group_norm(o_raw, x, skip, z, weight, groups, eps, out, row_slot, num_heads, v_dim):
    n, d = o_raw.shape
    zf = z.to(torch.float32)
    y = (o_raw + skip.repeat_interleave(v_dim)[None, :] * x.to(torch.float32)) * (zf * torch.sigmoid(zf))
    parts = y.view(n, groups, d // groups)
    y = (parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, d) * weight
    out[:] = y.to(out.dtype)
    return out


def embed_pairs(table, pairs, tokens, positions, row_slot, row_last, prev, out, scale, buckets, mul_prev, mul_cur):
    toks = [int(t) for t in tokens]
    for r0, rows, slot in _segments(row_slot):
        for r in range(r0, r0 + rows):
            before = toks[r - 1] if r > r0 else (int(prev[slot, 0]) if int(positions[r]) > 0 else None)
            which = buckets if before is None else (before * mul_prev + toks[r] * mul_cur) % buckets
            out[r] = table[toks[r]].to(torch.float32) * scale + pairs[which].to(torch.float32)
        prev[slot, 0] = toks[r0 + rows - 1]
    return out


def group_norm(residual, delta_a, delta_b, groups, eps, w1, out1, w2=None, out2=None, in_place=False, dtype=None):
    for d in (delta_a, delta_b):
        if d is not None:
            residual += d.to(torch.float32)
    if w1 is None:
        return out1, out2
    n, width = residual.shape
    parts = residual.view(n, groups, width // groups)
    normed = (parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, width)
    if in_place:
        residual.copy_(normed * w1)
    elif out1 is not None:
        out1[:] = (normed * w1).to(out1.dtype)
    if out2 is not None:
        out2[:] = (normed * w2).to(out2.dtype)
    return out1, out2


def rotate_tie_store(qk, num_heads, kv_heads, dim, rot, cos, sin, k_pages, v_pages, block_table, positions, row_slot,
                     page_size, fault):
    half = rot // 2

    def turn(z, pos):                   # (heads, dim)
        if not rot:
            return z
        c, s = cos[pos], sin[pos]
        a, b = z[:, :half], z[:, half:rot]
        return torch.cat([a * c - b * s, b * c + a * s, z[:, rot:]], dim=-1)

    for r in range(qk.shape[0]):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        row = qk[r].to(torch.float32)
        q = row[:num_heads * dim].view(num_heads, dim)
        k = row[num_heads * dim:(num_heads + kv_heads) * dim].view(kv_heads, dim)
        qk[r, :num_heads * dim] = turn(q, pos).reshape(-1).to(qk.dtype)
        page = int(block_table[slot, pos // page_size])
        k_pages[page, :, pos % page_size, :] = turn(k, pos).to(k_pages.dtype)
        v_pages[page, :, pos % page_size, :] = k.to(v_pages.dtype)


def scaled_sum(a, scale_a, b, scale_b):
    return (a.to(torch.float32) * scale_a + b.to(torch.float32) * scale_b).to(a.dtype)


def moe_down(hidden, chosen, weights, w_down, shared, shared_gate):
    n, top = chosen.shape
    h = hidden.to(torch.float32).view(n, top, -1)
    y = torch.einsum("ntdf,ntf->ntd", w_down.to(torch.float32)[chosen.long()], h)
    out = (y * weights[:, :, None]).sum(1)
    if shared is not None:
        out = out + shared_gate[:, None] * shared.to(torch.float32)
    return out.to(hidden.dtype)


def residual_add(residual, delta):
    residual += delta.to(torch.float32)
    return residual


def _rotate(x, cos, sin, interleaved):
    """x (heads, hd) float32; cos, sin (rot/2,)."""
    rot = 2 * cos.shape[0]
    y = x.clone()
    if interleaved:
        a, b = x[:, 0:rot:2], x[:, 1:rot:2]
        y[:, 0:rot:2] = a * cos - b * sin
        y[:, 1:rot:2] = b * cos + a * sin
    else:
        h = rot // 2
        a, b = x[:, :h], x[:, h:rot]
        y[:, :h] = a * cos - b * sin
        y[:, h:rot] = b * cos + a * sin
    return y


def _chunk_places(nch, positions):
    """physical chunk of logical chunk c for rows at ``positions``: (L, nch).  Rows of a multiple
    of eight chunks: c XOR (position mod 8); other rows: (c + position) mod chunks."""
    c = torch.arange(nch)[None, :]
    pos = torch.as_tensor(positions).reshape(-1, 1)
    return (c ^ (pos & 7)) if nch % 8 == 0 else (c + pos) % nch


def cache_row(x, pos):
    """The cache's row format: a row of keys or values (last axis: head size) is stored as
    16-byte chunks permuted by the position."""
    n = 16 // x.element_size()
    hd = x.shape[-1]
    place = _chunk_places(hd // n, [pos])[0]
    chunks = x.reshape(*x.shape[:-1], hd // n, n)
    out = torch.empty_like(chunks)
    out[..., place, :] = chunks
    return out.reshape(x.shape)


def cache_row_inverse(x, pos):
    n = 16 // x.element_size()
    hd = x.shape[-1]
    place = _chunk_places(hd // n, [pos])[0]
    return x.reshape(*x.shape[:-1], hd // n, n)[..., place, :].reshape(x.shape)


def rope_kv_write(qkv, positions, row_slot, cos, sin, plane, block_table, num_heads, kv_heads, head_dim,
                  page_size, fault, interleaved=False, write_kv=True):
    n = qkv.shape[0]
    hq, hkv = num_heads * head_dim, kv_heads * head_dim
    for r in range(n):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        pos = int(positions[r])
        c, s = cos[pos], sin[pos]
        q = qkv[r, :hq].to(torch.float32).view(num_heads, head_dim)
        qkv[r, :hq] = _rotate(q, c, s, interleaved).reshape(-1).to(qkv.dtype)
        if not (write_kv and plane is not None):
            continue
        page = int(block_table[slot, pos // page_size])
        if page < 0 or page >= plane.shape[0]:
            fault[0] = 1
            continue
        k = qkv[r, hq:hq + hkv].to(torch.float32).view(kv_heads, head_dim)
        v = qkv[r, hq + hkv:hq + 2 * hkv].view(kv_heads, head_dim)
        plane[page, 0, :, pos % page_size, :] = cache_row(_rotate(k, c, s, interleaved).to(plane.dtype), pos)
        plane[page, 1, :, pos % page_size, :] = cache_row(v.to(plane.dtype), pos)


def gather_kv(plane, block_table, slot, lo, hi, page_size):
    """Keys and values lo..hi-1 of a slot: (hi-lo, KVH, hd) each, float32."""
    idx = torch.arange(lo, hi)
    pages = block_table[slot, (idx // page_size)].long()
    k = _unrotate_rows(plane[pages, 0, :, idx % page_size, :], idx)
    v = _unrotate_rows(plane[pages, 1, :, idx % page_size, :], idx)
    return k.to(torch.float32), v.to(torch.float32)


def _unrotate_rows(x, positions):
    """x (L, KVH, hd) as stored, row i belonging to positions[i]: back to logical order."""
    n = 16 // x.element_size()
    L, kvh, hd = x.shape
    nch = hd // n
    chunks = x.reshape(L, kvh, nch, n).permute(0, 2, 1, 3)                       # (L, nch, KVH, n)
    phys = _chunk_places(nch, positions)                                         # logical c -> physical chunk
    out = chunks[torch.arange(L)[:, None], phys]                                 # (L, nch, KVH, n)
    return out.permute(0, 2, 1, 3).reshape(L, kvh, hd)


def rotary_fusable(q, step, num_heads, kv_heads, head_dim):
    """On the CPU every decode step takes the path where attention does the rotary encoding and the
    cache write itself, so that its plumbing runs in the CPU tests too."""
    return step is not None and getattr(step, "decode_only", False)


def paged_attention(q, out, plane, block_table, positions, row_slot, num_heads, kv_heads, head_dim, page_size,
                    window, fault, step=None, rotary=None, write_kv=True):
    if rotary is not None:
        rope_kv_write(q, positions, row_slot, rotary[0], rotary[1], plane, block_table, num_heads, kv_heads, head_dim,
                      page_size, fault, write_kv=write_kv)
    n = q.shape[0]
    g = num_heads // kv_heads
    hq = num_heads * head_dim
    for r in range(n):
        slot = int(row_slot[r])
        if slot < 0:
            out[r] = 0
            continue
        pos = int(positions[r])
        hi = pos + 1
        lo = max(0, hi - window) if window else 0
        k, v = gather_kv(plane, block_table, slot, lo, hi, page_size)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        qq = q[r, :hq].to(torch.float32).view(num_heads, head_dim)
        s = torch.einsum("hd,khd->hk", qq, k) / math.sqrt(head_dim)
        p = torch.softmax(s, dim=-1)
        out[r] = torch.einsum("hk,khd->hd", p, v).reshape(-1).to(out.dtype)
    return out


def swiglu(gu, out, block=None):
    f = out.shape[1]
    block = block or f
    both = gu.to(torch.float32).reshape(gu.shape[0], f // block, 2, block)
    g = both[:, :, 0, :].reshape(-1, f)
    u = both[:, :, 1, :].reshape(-1, f)
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))
    return out


def gemm_swiglu(a, w_gu, hidden, block):
    gu = gemm(a, w_gu)
    return swiglu(gu, torch.empty((a.shape[0], hidden), dtype=a.dtype), block)


def mtp_input(h_prev, state, row_slot, row_last, tokens, table, scale, eps, out):
    n, d = h_prev.shape
    new_state = {}
    for r in range(n):
        slot = int(row_slot[r])
        if slot < 0:
            continue
        first = r == 0 or int(row_slot[r - 1]) != slot
        if first:
            out[r, :d] = state[slot]
            new_state[slot] = h_prev[int(row_last[r])].clone()
        else:
            out[r, :d] = h_prev[r - 1]
        e = table[int(tokens[r])].to(torch.float32)
        norm = e.pow(2).sum().sqrt()
        out[r, d:] = (e * math.sqrt(d) / (norm + eps) * scale).to(out.dtype)
    for slot, row in new_state.items():
        state[slot] = row
    return out


def _philox_u32(seed: int, counter: int) -> int:
    m0, m1 = 0xD2511F53, 0xCD9E8D57
    c = [counter & 0xFFFFFFFF, (counter >> 32) & 0xFFFFFFFF, 0, 0]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = m0 * c[0], m1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c[0]


def row_probs(logits_row, temp, top_k, top_p, penalty, seen_tokens):
    """Probabilities of one row as the sampling kernel defines them: all entries equal to a
    threshold value are kept."""
    x = logits_row.to(torch.float64).clone()
    if penalty != 1.0 and len(seen_tokens):
        idx = torch.tensor(sorted(set(int(t) for t in seen_tokens)), dtype=torch.long)
        x[idx] = torch.where(x[idx] > 0, x[idx] / penalty, x[idx] * penalty)
    x = x / temp
    v = x.shape[0]
    keep = torch.ones(v, dtype=torch.bool)
    if 0 < top_k < v:
        thr = torch.sort(x, descending=True).values[top_k - 1]
        keep &= x >= thr
    if 0 < top_p < 1:
        xs = torch.where(keep, x, torch.full_like(x, float("-inf")))
        p = torch.softmax(xs, -1)
        srt, _ = torch.sort(p, descending=True)
        cum = torch.cumsum(srt, -1)
        first_over = int((cum > top_p).nonzero()[0]) if bool((cum > top_p).any()) else v - 1
        keep &= p >= srt[first_over]
    xs = torch.where(keep, x, torch.full_like(x, float("-inf")))
    return torch.softmax(xs, -1)


def sample_rows(logits, temps, top_ks, top_ps, penalties, slots, seen_bitmap, seeds, counters, out_tokens,
                probs_out=None):
    k, v = logits.shape
    for r in range(k):
        temp, top_k = float(temps[r]), int(top_ks[r])
        slot = int(slots[r]) if slots is not None else -1
        seen = []
        if slot >= 0 and seen_bitmap is not None:
            words = seen_bitmap[slot]
            seen = [i for i in range(v) if (int(words[i >> 5]) >> (i & 31)) & 1]
        pen = float(penalties[r])
        greedy = not (temp > 0) or top_k == 1
        if greedy:
            x = logits[r].to(torch.float64).clone()
            if pen != 1.0 and seen:
                idx = torch.tensor(seen, dtype=torch.long)
                x[idx] = torch.where(x[idx] > 0, x[idx] / pen, x[idx] * pen)
            tok = int(torch.argmax(x))
            p = torch.zeros(v, dtype=torch.float64)
            p[tok] = 1
        else:
            p = row_probs(logits[r], temp, top_k, float(top_ps[r]), pen, seen)
            u = (_philox_u32(int(seeds[r]), int(counters[r])) >> 8) / 16777216.0
            cum = torch.cumsum(p, -1)
            over = (cum > u * float(cum[-1])) & (p > 0)
            tok = int(over.nonzero()[0]) if bool(over.any()) else int((p > 0).nonzero()[-1])
        out_tokens[r] = tok
        if probs_out is not None:
            probs_out[r] = p.to(torch.float32)
        if slot >= 0 and seen_bitmap is not None:
            w = int(seen_bitmap[slot, tok >> 5]) & 0xFFFFFFFF
            w |= 1 << (tok & 31)
            seen_bitmap[slot, tok >> 5] = w - (1 << 32) if w >= (1 << 31) else w
    return out_tokens


def bitmap_set(bitmap_row, tokens):
    for t in tokens.tolist():
        w = int(bitmap_row[t >> 5]) & 0xFFFFFFFF
        w |= 1 << (t & 31)
        bitmap_row[t >> 5] = w - (1 << 32) if w >= (1 << 31) else w


_NAMES = ["rotary_fusable", "gemm", "gemm_f32_out", "gemm_swiglu", "embed_rows", "add_rmsnorm", "residual_add", "rope_kv_write",
          "paged_attention", "swiglu", "mtp_input", "sample_rows", "bitmap_set", "glu_clamped", "scale_f32", "causal_conv",
          "softcap_f32", "activation", "gemm_act", "forget_gate_recurrence", "head_norm_store", "diff_combine",
          "norm_mix_store", "window_attention", "delta_rule", "linear_attention", "latent_prepare", "gemm_heads", "moe_route",
          "moe_gate_up", "moe_down", "moe_experts", "gated_linear_attention", "state_space_scan", "skip_gate_group_norm",
          "embed_pairs", "group_norm", "rotate_tie_store", "scaled_sum"]


def install(monkeypatch) -> None:
    """Put the references in place of the CUDA operations (CPU tests only)."""
    from tiny_inference_server_b200.kernels import ops

    g = globals()
    for name in _NAMES:
        monkeypatch.setattr(ops, name, g[name])
    monkeypatch.setattr(ops.ScaledRows, "dense", scaled_rows_dense)
