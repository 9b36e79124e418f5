"""Plain implementation of the Mivorax decoder for the tests: whole sequences, float64, no cache,
no batching, one function per mechanism. It shares no code with the package: it reads config.json
and the safetensors file itself and computes every layer from the equations given in each
function's docstring.
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


def embed_tokens(tokens, table, bigram, buckets, mul_prev, mul_cur):
    """x_t = table[tok_t] + bigram[r_t]; r_0 = buckets (the extra last row),
    r_t = (tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets for t > 0."""
    rows = []
    for t, tok in enumerate(tokens):
        r = buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets
        rows.append(table[tok] + bigram[r])
    return torch.stack(rows)


def rotate_half(x, positions, base, dims):
    """The first ``dims`` entries of the last dimension are rotated, the rest pass: entry i pairs with
    entry i + dims/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2 i / dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(F64)[:, None] * f[None, :]                 # [T, half]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def distance_bucket(n: int, rows: int, dmax: float) -> int:
    """Exact below rows/2, logarithmic above: the upper half of the table covers distances rows/2 .. dmax."""
    h = rows // 2
    if n < h:
        return n
    return min(rows - 1, h + int(math.floor(math.log(n / h) / math.log(dmax / h) * (rows - h))))


def softmax_attention(q, k, v, scale, bias=None, sink=None):
    """One head, causal. q [T, dk], k [T, dk], v [T, dv]; s_ij = scale q_i.k_j (+ bias_ij) for j <= i;
    p_ij = exp(s_ij) / (sum_j exp(s_ij) [+ exp(sink)]); out_i = sum_j p_ij v_j."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    if bias is not None:
        s = s + bias
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, torch.full_like(m, float(sink)))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - m)
    return (e / den) @ v


def biased_attention(h, w, p, mx):
    """Grouped-query attention without rotation; a learned bias rel[bucket(i - j), head] is added to the
    scaled scores."""
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, G, dk)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    idx = torch.tensor([[distance_bucket(i - j, rows, mx["bias_max"]) if j <= i else 0 for j in range(T)]
                        for i in range(T)])
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        outs.append(softmax_attention(q[:, hd], k[:, g], v[:, g], mx["scale"], bias=rel[:, hd][idx]))
    return torch.cat(outs, -1) @ w[p + "o"].T


def latent_attention(h, w, p, mx, eps):
    """Queries and keys/values through low-rank latents. c_q = norm(W_dq h); q = W_uq c_q, per head
    [dim plain | rot_dim rotated]. W_dkv h = [kv_rank latent | rot_dim]; c = norm(latent); the last rot_dim
    entries, rotated, are one key part that all heads share. Per head k = [W_uk c | shared part], v = W_uv c.
    The softmax denominator holds exp(sink_head) once more."""
    H, dk, dr, dv, rk = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, dk + dr)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :rk], w[p + "dkv.norm"], eps)
    rot = mx["rot"]
    k_rot = rotate_half(kv[:, rk:], pos, rot["base"], rot["dims"])
    q_rot = rotate_half(q[..., dk:], pos, rot["base"], rot["dims"])
    k_up = (c @ w[p + "uk"].T).view(T, H, dk)
    v_up = (c @ w[p + "uv"].T).view(T, H, dv)
    outs = []
    for hd in range(H):
        qh = torch.cat([q[:, hd, :dk], q_rot[:, hd]], -1)
        kh = torch.cat([k_up[:, hd], k_rot], -1)
        outs.append(softmax_attention(qh, kh, v_up[:, hd], mx["scale"], sink=w[p + "sink"][hd]))
    return torch.cat(outs, -1) @ w[p + "o"].T


def causal_conv(x, weight, bias):
    """Per channel: y_t = bias + sum_k weight[:, k] x_{t - (K - 1) + k}, zeros before the sequence."""
    T, C = x.shape
    K = weight.shape[1]
    xp = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    y = bias.expand(T, C).clone()
    for k in range(K):
        y = y + xp[k:k + T] * weight[:, k]
    return y


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def state_space_scan(x, B, C, dt, a_log, D, heads, groups):
    """Per head h with group g(h) = h // (heads / groups), state S [N, P] from zero:
    S_t = exp(-exp(a_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T;  y_t = S_t^T C_t + D_h x_t."""
    T = x.shape[0]
    P = x.shape[1] // heads
    N = B.shape[1] // groups
    x = x.view(T, heads, P)
    B = B.view(T, groups, N)
    C = C.view(T, groups, N)
    y = torch.zeros(T, heads, P, dtype=F64)
    for h in range(heads):
        g = h // (heads // groups)
        S = torch.zeros(N, P, dtype=F64)
        rate = torch.exp(a_log[h])
        for t in range(T):
            S = torch.exp(-rate * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y.reshape(T, heads * P)


def mamba2(h, w, p, mx, eps):
    """in -> [z | x | B | C | dt]; causal convolution + silu over [x | B | C]; dt = softplus(dt + dt_bias);
    the scan; y * silu(z), then RMS norm over ``norm_groups`` equal parts, times the norm weight; out."""
    heads, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = heads * P
    T = h.shape[0]
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x, B, C = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
    dt = softplus(dt + w[p + "dt_bias"])
    y = state_space_scan(x, B, C, dt, w[p + "A_log"], w[p + "D"], heads, G)
    y = y * silu(z)
    ng = mx["norm_groups"]
    y = rms_norm(y.view(T, ng, inner // ng), None, eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def dense_mlp(h, w, p):
    """down(relu(up h)^2)."""
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


# ---- the model ------------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] (float64) of one whole sequence; with ``return_layers`` also the residual stream
    after every layer run [runs, T, width]."""
    eps = cfg["norm"]["eps"]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg is None:
        x = torch.stack([w["embed"][t] for t in tokens])
    else:
        x = embed_tokens(list(tokens), w["embed"], w["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        src = i if src is None else src
        p = f"l{src}."
        hn = rms_norm(x, w[p + "norm1"], eps)
        kind, mx = layer["type"], layer["mixer"]
        if kind == "attention":
            x = x + biased_attention(hn, w, p + "mix.", mx)
        elif kind == "latent_attention":
            x = x + latent_attention(hn, w, p + "mix.", mx, eps)
        elif kind == "mamba2":
            x = x + mamba2(hn, w, p + "mix.", mx, eps)
        else:
            raise ValueError(f"layer type {kind!r}")
        if layer.get("mlp") is not None:
            x = x + dense_mlp(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        layers.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def generate(cfg, w, prompt, n_new):
    """Greedy continuation (ties to the lowest id)."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
