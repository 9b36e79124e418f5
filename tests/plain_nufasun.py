"""Plain implementation of the Nufasun decoder for the tests: whole sequences, float64, no cache, no batching,
one function per mechanism. It shares no code with the package: it reads config.json and the safetensors file
itself and computes every layer from the equations in each function's docstring.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ---- model folder ---------------------------------------------------------------------------

def read_model_folder(folder: str):
    """(config dictionary, {tensor name: float64 or int64 tensor})."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, ent in head.items():
        if name == "__metadata__":
            continue
        a, b = ent["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        dt = ent["dtype"]
        if dt == "BF16":
            u = raw.view("<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).astype(np.float64))
        elif dt == "F32":
            t = torch.from_numpy(raw.view("<f4").astype(np.float64))
        elif dt == "I32":
            t = torch.from_numpy(raw.view("<i4").astype(np.int64))
        else:
            raise ValueError(f"dtype {dt} of {name}")
        w[name] = t.reshape(ent["shape"])
    return cfg, w


# ---- mechanisms -----------------------------------------------------------------------------

def rms_norm(x, weight, eps):
    """y = x / sqrt(mean(x^2) + eps) * weight over the last dimension (weight None: no scaling)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_pairs(x, positions, base, dims):
    """The first ``dims`` entries of the last dimension are rotated in neighbouring pairs (2i, 2i + 1), the rest
    pass: (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2 i / dims). x is [T, ..., size]."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(F64)[:, None] * f[None, :]                 # [T, half]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def windowed_softmax_attention(q, k, v, scale, softcap, window):
    """One attention map of one head. q, k [T, dk], v [T, dv]. s_ij = cap * tanh(scale * q_i . k_j / cap) for
    0 <= i - j < window, softmax over those j, out_i = sum_j p_ij v_j. (No cap when ``softcap`` is 0 or None, every
    earlier token seen when ``window`` is None.)"""
    T = q.shape[0]
    s = (q @ k.t()) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if window is None else (j <= i) & (i - j < window)
    s = s.masked_fill(~seen, -math.inf)
    return torch.softmax(s, -1) @ v


def differential_attention(h, w, p, mx, eps):
    """The 'attention' mixer on the normed rows h [T, width]; w: tensors, p: their prefix ('l3.mix.').
    Per head two maps with queries and keys of their own over the same values:
        q[h, m], k[g, m]: RMS norm with a shared weight, then rotation of the first rot.dims entries
        a_m = windowed_softmax_attention(q[h, m], k[g, m], v[g]),  g = h // (heads / kv_heads)
        lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
        o_h = rms_norm(a_1 - lam a_2) (1 - diff) sigmoid(W_g h)_h
    out = W_o concat_h o_h."""
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].t()).view(T, H, 2, dk)
    k = (h @ w[p + "k"].t()).view(T, G, 2, dk)
    v = (h @ w[p + "v"].t()).view(T, G, dv)
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    if mx.get("rot") and mx["rot"]["dims"] > 0:
        q = rotate_pairs(q, pos, mx["rot"]["base"], mx["rot"]["dims"])
        k = rotate_pairs(k, pos, mx["rot"]["base"], mx["rot"]["dims"])
    window = mx["mask"]["size"] if mx.get("mask") else None
    lam = (torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum())
           + mx["diff"])
    gate = torch.sigmoid(h @ w[p + "g"].t())                    # [T, H]
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a = [windowed_softmax_attention(q[:, hh, m], k[:, g, m], v[:, g], mx["scale"], mx.get("softcap"), window)
             for m in range(2)]
        o = rms_norm(a[0] - lam * a[1], None, eps) * (1.0 - mx["diff"])
        heads.append(o * gate[:, hh:hh + 1])
    return torch.cat(heads, -1) @ w[p + "o"].t()


def causal_conv_silu(x, weight):
    """x [T, C], weight [C, taps]: y_t = silu(sum_k weight[:, k] x_{t - (taps - 1) + k}), zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for k in range(taps):
        y = y + xp[k:k + T] * weight[:, k][None, :]
    return y * torch.sigmoid(y)


def unit(x):
    """x / sqrt(sum(x^2) + 1e-6) over the last dimension."""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule_head(q, k, v, beta, decay):
    """One head of the gated delta rule, token by token. q, k [T, dk], v [T, dv], beta, decay [T]; S is dk x dv,
    zero at the start:  S <- decay_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, dk = q.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.t() @ q[t])
    return torch.stack(out)


def delta_mixer(h, w, p, mx, eps):
    """The 'delta' mixer on the normed rows h [T, width]: projections, short convolutions with silu, unit
    queries (times dk^-1/2) and keys, beta = sigmoid(W_b h), decay = exp(-exp(A_log) softplus(W_a h + dt_bias)),
    the recurrence per head (head hh reads q/k head hh // (heads / kv_heads)), then per head
    rms_norm(o) * norm * silu(W_g h), and W_o."""
    T = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = causal_conv_silu(h @ w[p + "q"].t(), w[p + "q.conv"]).view(T, G, dk)
    k = causal_conv_silu(h @ w[p + "k"].t(), w[p + "k.conv"]).view(T, G, dk)
    v = causal_conv_silu(h @ w[p + "v"].t(), w[p + "v.conv"]).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].t())                                     # [T, H]
    dt = torch.nn.functional.softplus(h @ w[p + "a"].t() + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)                           # [T, H]
    gate = (h @ w[p + "g"].t()).view(T, H, dv)
    gate = gate * torch.sigmoid(gate)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        o = delta_rule_head(q[:, g], k[:, g], v[:, hh], beta[:, hh], decay[:, hh])
        heads.append(rms_norm(o, w[p + "norm"], eps) * gate[:, hh])
    return torch.cat(heads, -1) @ w[p + "o"].t()


def limited_gated_feed_forward(h, w, p, limit):
    """g = min(W_gate h + b, limit), u = clamp(W_up h + b, -limit, limit),
    y = g sigmoid(1.702 g) (u + 1), out = W_down y + b."""
    g = torch.clamp(h @ w[p + "gate"].t() + w[p + "gate.b"], max=limit)
    u = torch.clamp(h @ w[p + "up"].t() + w[p + "up.b"], -limit, limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ w[p + "down"].t() + w[p + "down.b"]


def run_order(cfg):
    """[(layer, pass number or None, first of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


# ---- the model ------------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))] * cfg["embedding"]["scale"]
    x0 = x.clone()
    layers = []
    for i, t, first in run_order(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        layer = cfg["layers"][i]
        p = f"l{i}."
        hn = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            m = differential_attention(hn, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "delta":
            m = delta_mixer(hn, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(m, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            f = limited_gated_feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"]["limit"])
            x = x + rms_norm(f, w[p + "norm2b"], eps)
        layers.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].t()
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    if return_layers:
        return logits, torch.stack(layers)
    return logits


def greedy(cfg, w, prompt, n):
    """n greedy tokens after the prompt (each from a forward pass over the whole sequence so far)."""
    toks = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(forward(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
