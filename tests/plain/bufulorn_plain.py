"""The Bufulorn decoder written out plainly: one function per mechanism, whole sequences, token by
token where the mechanism is a recurrence, in whatever floating type the tensors have (the tests
use float64). Nothing here is shared with the engine: no kernel, no part, no cache.

Notation. x [T, width] is a sequence of T tokens at positions 0 .. T-1. A linear weight W is stored
[out, in] and applied as x W^T. `t` is the dictionary of tensors by name, `p` the prefix of a
mixer's or feed-forward's tensors, `m` its configuration.

The residual takes the NORMED result of each sub-layer: x += LN1(mixer(x)); x += LN2(ff(x)); the
sub-layers read x as it is.
"""
from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------------- small pieces
def layer_norm(z: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = z.mean(-1, keepdim=True)
    var = ((z - mu) ** 2).mean(-1, keepdim=True)
    return (z - mu) / torch.sqrt(var + eps) * w + b


def rms(z: torch.Tensor, eps: float) -> torch.Tensor:
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    zn = torch.clamp(z, max=0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(zn) - zn) + 0.5 * z)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------------- attention
def chunk_visible(T: int, size) -> torch.Tensor:
    """[T, T] bool: key j is seen from i when j <= i and both lie in the same block of `size`
    positions counted from 0 (no `size`: every earlier key)."""
    i = torch.arange(T)
    vis = i[None, :] <= i[:, None]
    if size:
        vis = vis & (torch.div(i, size, rounding_mode="floor")[None, :] == torch.div(i, size, rounding_mode="floor")[:, None])
    return vis


def attention_keys_values(h, t, p, m, eps):
    """The keys (after their norm) and values a layer leaves in its cache: [T, G, d], [T, G, dv]."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ t[p + "k"].T + t[p + "k.b"]).reshape(T, G, d)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).reshape(T, G, dv)
    return rms(k, eps) * t[p + "k.norm"], v


def chunk_attention(h, t, p, m, eps, kv=None):
    """Softmax attention inside blocks of positions: biased projections, q and k normed per head with a
    shared weight, score = cap * tanh(q.k * scale / cap) - r1_h ln(1 + r2_h (i - j)), a sigmoid gate
    from the same input on the heads' results. `kv`: keys and values of another layer to use instead
    of this layer's own. Returns (result, (keys, values))."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ t[p + "q"].T + t[p + "q.b"]).reshape(T, H, d), eps) * t[p + "q.norm"]
    k, v = kv if kv is not None else attention_keys_values(h, t, p, m, eps)
    kk, vv = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :]).clamp(min=0).to(h.dtype)
    s = s - t[p + "r1"][:, None, None] * torch.log1p(t[p + "r2"][:, None, None] * dist)
    vis = chunk_visible(T, (m.get("mask") or {}).get("size"))
    w = torch.softmax(s.masked_fill(~vis, -math.inf), dim=-1)
    o = torch.einsum("hij,jhd->ihd", w, vv).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ t[p + "g"].T)) @ t[p + "o"].T, (k, v)


# ----------------------------------------------------------------------------------- delta rule
def causal_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return silu(y)


def gated_delta(h, t, p, m, eps):
    """Gated delta rule with one decay per head. Per value head a state S [dim, vdim], zero at the start:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ t[p + "q"].T, t[p + "q.conv"]).reshape(T, G, d)
    k = causal_conv_silu(h @ t[p + "k"].T, t[p + "k.conv"]).reshape(T, G, d)
    v = causal_conv_silu(h @ t[p + "v"].T, t[p + "v.conv"]).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ t[p + "b"].T)                                              # [T, H]
    g = torch.exp(-torch.exp(t[p + "A_log"]) * softplus(h @ t[p + "a"].T + t[p + "dt_bias"]))   # [T, H]
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        S = g[i][:, None, None] * S
        u = beta[i][:, None] * (v[i] - torch.einsum("hkv,hk->hv", S, k[i]))
        S = S + k[i][:, :, None] * u[:, None, :]
        o[i] = torch.einsum("hkv,hk->hv", S, q[i])
    o = rms(o, eps) * t[p + "norm"] * silu(h @ t[p + "g"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ t[p + "o"].T


# ----------------------------------------------------------------------------------- feed-forward
def dense_ff(h, t, p):
    return xielu(h @ t[p + "up"].T, t[p + "act"][0], t[p + "act"][1]) @ t[p + "down"].T


def route(h, t, p, r):
    """Chosen experts [T, top] and their weights: softmax over all experts; the experts are cut into
    `groups.count` runs of neighbours, a run scores as its best expert, only experts of the best
    `groups.keep` runs stand for election; the `top` best of those, weighted by their own softmax
    scores as they are."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ t[p + "router"].T, dim=-1)                                     # [T, E]
    allowed = torch.ones_like(s, dtype=torch.bool)
    grp = r.get("groups")
    if grp:
        n, keep = grp["count"], grp["keep"]
        best = s.reshape(-1, n, E // n).max(-1).values                                   # [T, n]
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = kept.repeat_interleave(E // n, dim=1)
    idx = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def moe_ff(h, t, p, mlp):
    idx, w = route(h, t, p, mlp["router"])
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(mlp["router"]["experts"]):
        q = f"{p}e{e}."
        y = (silu(h @ t[q + "gate"].T) * (h @ t[q + "up"].T)) @ t[q + "down"].T
        out = out + y * ((idx == e).to(h.dtype) * w).sum(-1, keepdim=True)
    return out


# ----------------------------------------------------------------------------------- the model
def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence. `layers_out`, a list, receives the residual after every layer."""
    t = {n: (x.to(dtype) if x.is_floating_point() else x) for n, x in tensors.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = t["embed"][torch.tensor(list(tokens), dtype=torch.long)] + t["pos"][:T]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            y, kept[i] = chunk_attention(x, t, p + "mix.", m, eps, kept[src] if src is not None else None)
        elif layer["type"] == "delta":
            y = gated_delta(x, t, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, t[p + "norm1"], t[p + "norm1.b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(x, t, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, t, p + "mlp.", mlp)
            x = x + layer_norm(y, t[p + "norm2"], t[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, t["final.norm"], t["final.norm.b"], eps) @ t["head"].T
