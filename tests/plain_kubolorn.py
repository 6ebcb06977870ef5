"""Plain, slow implementation of the Kubolorn decoder: whole sequences, no cache, one function per
mechanism, ordinary tensor arithmetic in float64, token by token where the design is a recurrence.  It takes
the configuration as the dictionary of ``config.json`` and the weights as a dictionary of tensors by name (it
reads both on its own) and shares no code with the engine package.

Notation: ``L`` tokens of one sequence, ``t`` a position from 0, ``u`` the input of a sublayer, ``W[name]`` a
tensor stored ``(out, in)``.

* embedding: ``x_t = E[tok_t] * s + B[(tok_(t-1) * a + tok_t * b) mod n]`` (``B[n]`` for t = 0), then the
  model's norm;
* norm: the vector in ``g`` equal consecutive parts, each divided by its own root mean square, the whole times w;
* layer: ``x += mixer(u1) + ff(u2)`` with ``u_i = n_i + conv_i(n_i)``, ``n_i = norm_i(x)``: both sublayers read
  the same x, each through a norm and a short causal convolution of its own;
* mixers: ``gla`` (``gated_linear_attention``) and ``parallel`` (``sink_attention`` beside ``state_space_duality``);
* feed-forwards: ``dense_ff`` and ``expert_mixture``;
* a span of layers may run several times in a row with the same weights.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def read_config(folder: str) -> dict:
    import json
    import os
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=F64) -> dict:
    import os
    from safetensors.torch import load_file
    return {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def grouped_rms(z, groups: int, eps: float):
    """Every one of ``groups`` equal consecutive parts of the last dimension by its own root mean square."""
    parts = z.unflatten(-1, (groups, z.shape[-1] // groups))
    return (parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)).flatten(-2)


def short_conv(u, w, bias=None):
    """``y_t = sum_j w[:, j] * u_(t - taps + 1 + j)``; ``u`` (L, C), ``w`` (C, taps); zeros before t = 0."""
    L, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(L):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    if bias is not None:
        y = y + bias
    return y


# --------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------

def embed(c, W, tokens):
    e = c["embedding"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * e["scale"]
    b = e.get("bigram")
    if b:
        rows = []
        for t, tok in enumerate(tokens):
            rows.append(b["buckets"] if t == 0 else (int(tokens[t - 1]) * b["mul_prev"] + int(tok) * b["mul_cur"]) % b["buckets"])
        x = x + W["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


# --------------------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------------------

def gated_linear_attention(u, W, p, m, eps):
    """Per head ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``; alpha per key channel."""
    L = u.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (u @ W[p + "q"].T).view(L, H, D) * D ** -0.5
    k = (u @ W[p + "k"].T).view(L, H, D)
    v = (u @ W[p + "v"].T).view(L, H, V)
    z = (u @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(L, H, D)
    S = torch.zeros(H, D, V, dtype=u.dtype)
    o = torch.zeros(L, H, V, dtype=u.dtype)
    for t in range(L):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * W[p + "norm"]
    return (o.reshape(L, H * V) * silu(u @ W[p + "g"].T)) @ W[p + "o"].T


def rescaled_frequencies(rot):
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def channel(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(channel(sc["fast"])), 0)
    hi = min(math.ceil(channel(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(z, rot, first_position: int = 0):
    """``z`` (L, heads, dim): the first ``rot.dims`` channels of each head, channel i paired with i + dims/2."""
    dims = rot["dims"]
    f, mag = rescaled_frequencies(rot)
    ang = torch.arange(first_position, first_position + z.shape[0], dtype=F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    a, b = z[..., :dims // 2], z[..., dims // 2:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, z[..., dims:]], dim=-1)


def sink_attention(u, W, p, m):
    """Causal softmax attention whose values are the keys before rotation and whose denominator holds one more
    term ``exp(sink_h)``."""
    L = u.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (u @ W[p + "q"].T).view(L, H, D)
    k = (u @ W[p + "k"].T).view(L, G, D)
    v = k
    q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    out = torch.zeros(L, H, D, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(torch.ones(L, L, dtype=torch.bool).triu(1), float("-inf"))
        big = torch.maximum(s.max(-1).values, W[p + "sink"][h])
        e = torch.exp(s - big[:, None])
        out[:, h] = (e / (e.sum(-1) + torch.exp(W[p + "sink"][h] - big))[:, None]) @ v[:, g]
    return out.reshape(L, H * D) @ W[p + "o"].T


def state_space_duality(u, W, p, m, eps):
    """Per head ``S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T``, ``y_t = S_t^T C_t + D x_t``."""
    L = u.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = u @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(L, H, P)
    B = xbc[:, inner:inner + G * N].view(L, G, N)
    C = xbc[:, inner + G * N:].view(L, G, N)
    dt = torch.nn.functional.softplus(dt + W[p + "dt_bias"])
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * dt)
    S = torch.zeros(H, N, P, dtype=u.dtype)
    y = torch.zeros(L, H, P, dtype=u.dtype)
    for t in range(L):
        for h in range(H):
            g = h // (H // G)
            S[h] = decay[t, h] * S[h] + dt[t, h] * B[t, g][:, None] * x[t, h][None, :]
            y[t, h] = S[h].T @ C[t, g] + W[p + "D"][h] * x[t, h]
    y = y.reshape(L, inner) * silu(z)
    return (grouped_rms(y, m["norm_groups"], eps) * W[p + "norm"]) @ W[p + "o"].T


def side_by_side(u, W, p, m, eps):
    return m["left_scale"] * sink_attention(u, W, p + "left.", m["left"]) + \
        m["right_scale"] * state_space_duality(u, W, p + "right.", m["right"], eps)


MIXERS = {"gla": gated_linear_attention, "parallel": side_by_side}


# --------------------------------------------------------------------------------------
# feed-forwards
# --------------------------------------------------------------------------------------

def dense_ff(u, W, p, f):
    return gelu_tanh(u @ W[p + "up"].T) @ W[p + "down"].T


def expert_mixture(u, W, p, f):
    r = f["router"]
    logits = u @ W[p + "router"].T
    top = torch.topk(logits, r["top"], dim=-1)
    weights = torch.softmax(top.values, dim=-1)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(r["top"]):
            e = int(top.indices[t, j])
            out[t] += weights[t, j] * (relu_squared(u[t] @ W[f"{p}e{e}.up"].T) @ W[f"{p}e{e}.down"].T)
    return out


def feed_forward(u, W, p, f):
    return dense_ff(u, W, p, f) if f["kind"] == "dense" else expert_mixture(u, W, p, f)


# --------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------

def layer_runs(c):
    """The layers in running order: the looped span several times in a row."""
    n = len(c["layers"])
    loop = c.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def plain_forward(c: dict, W: dict, tokens, return_layers: bool = False):
    eps, groups = c["norm"]["eps"], c["norm"].get("groups", 1)
    canon = (c.get("canon") or {}).get("taps")
    x = grouped_rms(embed(c, W, tokens), groups, eps) * W["embed.norm"]
    layers = []
    for i in layer_runs(c):
        layer, p = c["layers"][i], f"l{i}."
        u = grouped_rms(x, groups, eps) * W[p + "norm1"]
        if canon:
            u = u + short_conv(u, W[p + "canon1"])
        delta = MIXERS[layer["type"]](u, W, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            u = grouped_rms(x, groups, eps) * W[p + "norm2"]
            if canon:
                u = u + short_conv(u, W[p + "canon2"])
            delta = delta + feed_forward(u, W, p + "mlp.", layer["mlp"])
        x = x + delta
        layers.append(x.clone())
    logits = (grouped_rms(x, groups, eps) * W["final.norm"]) @ W["embed"].T
    if return_layers:
        return logits, torch.stack(layers)
    return logits
