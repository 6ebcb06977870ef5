"""Plain, slow implementation of the Biruvik decoder: whole sequences, no cache, one function per
mechanism, ordinary tensor arithmetic in float64.  It reads ``config.json`` and ``model.safetensors``
on its own and shares no code with the engine package.

Notation: ``L`` tokens of one sequence, ``t`` a position from 0, ``u`` the input of a sublayer (the
residual stream after the sublayer's first norm), ``W[name]`` a tensor stored ``(out, in)``;
``rms(z) = z * (mean(z^2) + eps)^-1/2``.

* stream: ``x_t = E[token_t] * s_e``; every layer ``x += g1b * rms(mixer(g1 * rms(x)))`` and, if the layer
  has a feed-forward, ``x += g2b * rms(ff(g2 * rms(x)))``: a norm in front of and behind every sublayer, each
  with ONE number as its weight; logits ``cap * tanh(head @ (g_f * rms(x)) / cap)``.
* mixer ``attention``: every head runs two softmax maps over the same values and subtracts one from the
  other (``differential_attention``); queries grow with the logarithm of the position.
* mixer ``latent_attention``: keys and values of all heads are expanded from one small normed vector per
  token; a sliding window; one sigmoid gate per head (``latent_window_attention``).
* mixer ``hgrn2``: a matrix state per head whose forget gate, per key channel, also is one minus the key
  (``gated_forget_recurrence``).
* feed-forward: ``W_down act(W_up u)`` (``dense_ff``).
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=F64) -> dict:
    from safetensors.torch import load_file
    return {k: v.to(dtype) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------------------
# small pieces
# --------------------------------------------------------------------------------------

def rms(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


ACTIVATIONS = {"relu2": relu_squared, "gelu_tanh": gelu_tanh, "silu": silu}


def softmax_rows(scores, visible):
    """scores (..., L, L), visible (L, L) bool: softmax over the visible keys of every row."""
    return torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)


def causal(L):
    i = torch.arange(L)
    return i[:, None] >= i[None, :]


def banded(L, size):
    """Row i sees j with 0 <= i - j < size."""
    i = torch.arange(L)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


# --------------------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------------------

def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1): constant over runs of ``every`` positions."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(F64)
    return 1.0 + coef * torch.log(steps + 1.0)


def differential_lambda(W, p, diff):
    return (torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum()) + diff).item()


def differential_attention(u, W, p, m, eps, positions=None):
    L = u.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(L) if positions is None else positions
    q = (u @ W[p + "q"].T + W[p + "q.b"]).view(L, H, 2, dim)
    k = (u @ W[p + "k"].T + W[p + "k.b"]).view(L, G, 2, dim)
    v = (u @ W[p + "v"].T + W[p + "v.b"]).view(L, G, vdim)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(pos, temp["coef"], temp["every"]).view(L, 1, 1, 1)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihmd,jhmd->hmij", q, k) * m["scale"]
    mask = m.get("mask")                                               # a window, if the layer has one; else every j <= i
    w = softmax_rows(s, banded(L, mask["size"]) if mask else causal(L))   # (H, 2, L, L)
    a = torch.einsum("hmij,jhd->imhd", w, v)                           # both maps read the same values
    lam = differential_lambda(W, p, m["diff"])
    o = rms(a[:, 0] - lam * a[:, 1], eps) * (1.0 - m["diff"])          # per head over vdim, no weight
    return o.reshape(L, H * vdim) @ W[p + "o"].T


def latent_window_attention(u, W, p, m, eps):
    L = u.shape[0]
    H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = (u @ W[p + "q"].T).view(L, H, dim)
    c = rms(u @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]               # (L, rank): all a cache would hold
    k = (c @ W[p + "uk"].T).view(L, H, dim)
    v = (c @ W[p + "uv"].T).view(L, H, vdim)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = m.get("mask")
    w = softmax_rows(s, banded(L, mask["size"]) if mask else causal(L))
    o = torch.einsum("hij,jhd->ihd", w, v)
    o = o * torch.sigmoid(u @ W[p + "g"].T)[:, :, None]                # one gate per head
    return o.reshape(L, H * vdim) @ W[p + "o"].T


def gated_forget_recurrence(u, W, p, m, eps, state=None):
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T; o_t = S_t^T q_t.  ``state`` (H, dim, vdim): where to start."""
    L = u.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(u @ W[p + "q"].T).view(L, H, dim)
    v = (u @ W[p + "v"].T).view(L, H, vdim)
    low = W[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(u @ W[p + "f"].T + W[p + "f.b"])).view(L, H, dim)
    S = torch.zeros((H, dim, vdim), dtype=u.dtype) if state is None else state.clone()
    o = torch.zeros((L, H, vdim), dtype=u.dtype)
    for t in range(L):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * W[p + "norm"]
    return o.reshape(L, H * vdim) @ W[p + "o"].T


# --------------------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------------------

def dense_ff(u, W, p, f):
    act = ACTIVATIONS[f.get("act", "relu2")]
    return act(u @ W[p + "up"].T) @ W[p + "down"].T


# --------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------

MIXERS = {"attention": differential_attention, "latent_attention": latent_window_attention,
          "hgrn2": gated_forget_recurrence}


def plain_forward(c: dict, W: dict, tokens, return_layers: bool = False):
    eps = c["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (c.get("embedding") or {}).get("scale", 1.0)
    layers = []
    for i, layer in enumerate(c["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](rms(x, eps) * W[p + "norm1"], W, p + "mix.", layer["mixer"], eps)
        x = x + rms(y, eps) * W[p + "norm1b"]
        if layer.get("mlp"):
            y = dense_ff(rms(x, eps) * W[p + "norm2"], W, p + "mlp.", layer["mlp"])
            x = x + rms(y, eps) * W[p + "norm2b"]
        layers.append(x.clone())
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T
    cap = c.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    if return_layers:
        return logits, torch.stack(layers)
    return logits
