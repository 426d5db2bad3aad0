"""The Pironex decoder written out plainly: one function per mechanism, whole sequences, token by
token where the mechanism is a recurrence, in whatever floating type the tensors have (the tests
use float64). Nothing here is shared with the engine: no kernel, no part, no cache.

Notation. x [T, width] is a sequence of T tokens at positions 0 .. T-1. A linear weight W is stored
[out, in] and applied as x W^T. `t` is the dictionary of tensors by name, `p` the prefix of a
mixer's or feed-forward's tensors, `m` its configuration (config.json's own keys).

A layer:  x += LNb1(mixer(canon1(LN1(x))));  x += LNb2(ff(canon2(LN2(x))));  canon(h) = h + conv(h).
Between layers the stream is a learned weighted sum of the embedding and of every layer's result so far.
"""
from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------------- small pieces
def layer_norm(z, w, eps):
    mu = z.mean(-1, keepdim=True)
    var = ((z - mu) ** 2).mean(-1, keepdim=True)
    return (z - mu) / torch.sqrt(var + eps) * w


def rms(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(h, w, bias=None):
    """out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start. h [T, C], w [C, taps]."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            out[shift:] += h[:T - shift] * w[:, j]
    return out + bias if bias is not None else out


def canon(h, w):
    return h + causal_conv(h, w)


def rotate_half(x, pos, dims, base):
    """x [T, heads, d]: feature i pairs with i + dims/2 on the first `dims` features; the rest pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = pos.to(x.dtype)[:, None, None] * f
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def rotate_interleaved(x, pos, dims, base):
    """x [T, heads, d]: feature 2i pairs with 2i + 1 on the first `dims` features."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = pos.to(x.dtype)[:, None, None] * f
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------- attention with pooled blocks
def attention_keys_values(h, t, p, m, eps):
    """What the layer's cache holds: keys after the norm over the whole projection and the rotation, values."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rms(h @ t[p + "k"].T, eps) * t[p + "k.norm"]
    k = rotate_half(k.reshape(T, G, d), torch.arange(T), m["rot"]["dims"], m["rot"]["base"]) if m.get("rot") else k.reshape(T, G, d)
    v = (h @ t[p + "v"].T).reshape(T, G, dv)
    return k, v


def pooled_window_attention(q, k, v, scale, softcap, size, pool, rows=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]. Row i sees the tokens j with 0 <= i - j < size and, for each
    block b of `pool` tokens that ends at or before i - size, the mean of the block's keys with the mean of its values.
    `rows`: only these rows are worked out (the others stay zero)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in (range(T) if rows is None else rows):
        lo = max(0, i - size + 1) if size else 0
        ks, vs = [k[j] for j in range(lo, i + 1)], [v[j] for j in range(lo, i + 1)]
        if size and pool:
            b = 0
            while b * pool + pool - 1 <= i - size:
                ks.append(k[b * pool:(b + 1) * pool].mean(0))
                vs.append(v[b * pool:(b + 1) * pool].mean(0))
                b += 1
        K, V = torch.stack(ks), torch.stack(vs)                       # [n, G, d]
        for hh in range(H):
            g = hh // (H // G)
            s = (K[:, g] @ q[i, hh]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            out[i, hh] = torch.softmax(s, 0) @ V[:, g]
    return out


def attention_mixer(h, t, p, m, eps, kv=None):
    """`kv`: the keys and values of the layer this one reads (`kv_from`), else its own."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    q = rms(h @ t[p + "q"].T, eps) * t[p + "q.norm"]
    q = q.reshape(T, H, d)
    if m.get("rot"):
        q = rotate_half(q, torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    k, v = kv if kv is not None else attention_keys_values(h, t, p, m, eps)
    mask = m.get("mask") or {}
    o = pooled_window_attention(q, k, v, m["scale"], m.get("softcap") or 0.0, mask.get("size", 0), mask.get("pool", 0))
    return o.reshape(T, -1) @ t[p + "o"].T


# ----------------------------------------------------------------------------------- mamba2
def mamba2_mixer(h, t, p, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ t[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N].clone(), proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, t[p + "conv"], t[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + t[p + "dt_bias"])                              # [T, H]
    decay = torch.exp(-torch.exp(t[p + "A_log"]) * dt)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for i in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = decay[i, hh] * S[hh] + dt[i, hh] * torch.outer(B[i, g], x[i, hh])
            y[i, hh] = S[hh].T @ C[i, g] + t[p + "D"][hh] * x[i, hh]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


# ----------------------------------------------------------------------------------- latent attention
def latent_mixer(h, t, p, m, eps):
    T = h.shape[0]
    H, d, r, dv, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    pos = torch.arange(T)
    q = (h @ t[p + "q"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_interleaved(q[..., d:], pos, r, base)
    dkv = h @ t[p + "dkv"].T
    c = rms(dkv[:, :L], eps) * t[p + "dkv.norm"]
    k_rot = rotate_interleaved(dkv[:, None, L:], pos, r, base)[:, 0]   # [T, r], shared by the heads
    k_plain = (c @ t[p + "uk"].T).reshape(T, H, d)
    v = (c @ t[p + "uv"].T).reshape(T, H, dv)
    size = (m.get("mask") or {}).get("size", 0)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - size + 1) if size else 0
        for hh in range(H):
            s = (k_plain[lo:i + 1, hh] @ q_plain[i, hh] + k_rot[lo:i + 1] @ q_rot[i, hh]) * m["scale"]
            out[i, hh] = torch.softmax(s, 0) @ v[lo:i + 1, hh]
    return out.reshape(T, -1) @ t[p + "o"].T


# ----------------------------------------------------------------------------------- feed-forward
def clamped_expert(h, wg, wu, wd, limit):
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ wd.T


def moe(h, t, p, m):
    E, top = m["router"]["experts"], m["router"]["top"]
    z = h @ t[p + "router"].T
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for c in range(top):
            e = int(idx[i, c])
            out[i] += w[i, c] * clamped_expert(h[i:i + 1], t[f"{p}e{e}.gate"], t[f"{p}e{e}.up"], t[f"{p}e{e}.down"],
                                               m["expert"]["limit"])[0]
    if m.get("shared"):
        s = clamped_expert(h, t[p + "shared.gate"], t[p + "shared.up"], t[p + "shared.down"], m["shared"]["limit"])
        out = out + s * torch.sigmoid(h @ t[p + "shared.sg"].T)
    return out


# ----------------------------------------------------------------------------------- the model
def forward(cfg: dict, t: dict, tokens, dtype=None, layers_out=None):
    """tokens: list of ints -> logits [T, vocab]. `layers_out` (a list) receives the stream that every layer hands on."""
    if dtype is not None:
        t = {k: v.to(dtype) if v.is_floating_point() else v for k, v in t.items()}
    eps = cfg["norm"]["eps"]
    x = t["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    results = [x]
    kvs = {}
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        has_canon = cfg.get("canon") is not None
        h = layer_norm(x, t[pre + "norm1"], eps)
        if has_canon:
            h = canon(h, t[pre + "canon1"])
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kvs[i] = attention_keys_values(h, t, pre + "mix.", m, eps)
            y = attention_mixer(h, t, pre + "mix.", m, eps, kvs[i if src is None else src])
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(h, t, pre + "mix.", m, eps)
        else:
            y = latent_mixer(h, t, pre + "mix.", m, eps)
        x = x + layer_norm(y, t[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, t[pre + "norm2"], eps)
            if has_canon:
                h = canon(h, t[pre + "canon2"])
            x = x + layer_norm(moe(h, t, pre + "mlp.", layer["mlp"]), t[pre + "norm2b"], eps)
        results.append(x)
        w = t[pre + "dwa"]
        x = sum(w[j] * results[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    return layer_norm(x, t["final.norm"], eps) @ t["embed"].T
