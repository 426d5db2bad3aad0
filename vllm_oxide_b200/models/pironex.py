"""The Pironex decoder as a list of parts.

embedding times a constant; then the layers in order, each a `SandwichBlock` (a layer norm with a weight in front of
and behind each sub-layer; what a sub-layer reads first passes a short causal convolution that is added to it; the
stream handed to the next layer is a learned weighted sum of the embedding's output and every layer's result so far)
whose mixer is a `SoftmaxAttention` (a norm over the whole q and k projections, partial rotary positions, capped
scores, a window beside which blocks of tokens are seen pooled; with `kv_from` it reads the cache of an earlier layer
and has no key and value tensors), a `StateSpace` mixer or a `LatentAttention` in a window with the interleaved
pairing, and whose feed-forward is `RoutedExperts` with the clamped gate and a shared expert, or absent; then the model's
layer norm and the head, which is the embedding table itself.

Tensor names are the checkpoint's own: `embed`, `final.norm`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`,
`l<i>.canon1|canon2`, `l<i>.dwa`, `l<i>.mix.*` (`q k v o q.norm k.norm`; or `in conv conv.b dt_bias A_log D norm o`; or
`q dkv dkv.norm uk uv o`), `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`, `l<i>.mlp.shared.gate|up|down|sg`.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.pironex_config import NAME, PironexConfig
from ..config.registry import Architecture, register_architecture
from ..parts import Embedding, LayerCall, LMHead, ModelSpec
from ..parts.block import SandwichBlock
from ..parts.flex_attention import SoftmaxAttention
from ..parts.latent_attention import LatentAttention
from ..parts.layernorm import LayerNorm
from ..parts.moe import RoutedExperts
from ..parts.recurrent import StateSpace
from ..weights.loader import TensorSpec, WeightSet

DEPTH_STACK = "depth_stack"


def pironex_manifest(cfg: PironexConfig) -> Dict[str, TensorSpec]:
    w = cfg.width
    m = {"embed": TensorSpec((cfg.vocab, w))}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        x = p + "mix."
        m[p + "norm1"], m[p + "norm1b"] = TensorSpec((w,), init="ones"), TensorSpec((w,), init="ones")
        if cfg.canon_taps:
            m[p + "canon1"] = TensorSpec((w, cfg.canon_taps))
        if layer.type == "attention":
            a = layer.attention
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            m[x + "q"], m[x + "q.norm"] = TensorSpec((nq, w)), TensorSpec((nq,), init="ones")
            if a.kv_from is None:
                m[x + "k"], m[x + "k.norm"], m[x + "v"] = TensorSpec((nk, w)), TensorSpec((nk,), init="ones"), TensorSpec((nv, w))
            m[x + "o"] = TensorSpec((w, a.heads * a.vdim))
        elif layer.type == "mamba2":
            s = layer.ssm
            inner, chans = s.heads * s.vdim, s.heads * s.vdim + 2 * s.groups * s.state
            m[x + "in"] = TensorSpec((inner + chans + s.heads, w))
            m[x + "conv"], m[x + "conv.b"] = TensorSpec((chans, s.conv)), TensorSpec((chans,), init="zeros")
            m[x + "dt_bias"], m[x + "A_log"], m[x + "D"] = TensorSpec((s.heads,)), TensorSpec((s.heads,)), TensorSpec((s.heads,), init="ones")
            m[x + "norm"], m[x + "o"] = TensorSpec((inner,), init="ones"), TensorSpec((w, inner))
        else:
            c = layer.latent
            m[x + "q"] = TensorSpec((c.heads * (c.dim + c.rot_dim), w))
            m[x + "dkv"], m[x + "dkv.norm"] = TensorSpec((c.kv_rank + c.rot_dim, w)), TensorSpec((c.kv_rank,), init="ones")
            m[x + "uk"], m[x + "uv"] = TensorSpec((c.heads * c.dim, c.kv_rank)), TensorSpec((c.heads * c.vdim, c.kv_rank))
            m[x + "o"] = TensorSpec((w, c.heads * c.vdim))
        f = layer.mlp
        if f is not None:
            m[p + "norm2"], m[p + "norm2b"] = TensorSpec((w,), init="ones"), TensorSpec((w,), init="ones")
            if cfg.canon_taps:
                m[p + "canon2"] = TensorSpec((w, cfg.canon_taps))
            y = p + "mlp."
            m[y + "router"] = TensorSpec((f.experts, w))
            for e in range(f.experts):
                m[f"{y}e{e}.gate"], m[f"{y}e{e}.up"], m[f"{y}e{e}.down"] = TensorSpec((f.ff, w)), TensorSpec((f.ff, w)), TensorSpec((w, f.ff))
            if f.shared_ff:
                m[y + "shared.gate"], m[y + "shared.up"] = TensorSpec((f.shared_ff, w)), TensorSpec((f.shared_ff, w))
                m[y + "shared.down"], m[y + "shared.sg"] = TensorSpec((w, f.shared_ff)), TensorSpec((1, w))
        m[p + "dwa"] = TensorSpec((i + 2,), init="ones")
    m["final.norm"] = TensorSpec((w,), init="ones")
    return m


def _cache_keep(cfg: PironexConfig, j: int):
    """What the cache that layer j writes must keep for all the layers that read it: their common window when none of them
    looks behind it, else everything."""
    users = [cfg.layers[i].attention for i in cfg.cache_users(j)]
    if any(a.pool or not a.window for a in users) or len({a.window for a in users}) != 1:
        return ("full", 0)
    return ("window", users[0].window)


def _pooled_sizes(cfg: PironexConfig, j: int):
    """The block sizes the cache that layer j writes must serve: those of all the layers that read it."""
    return tuple(sorted({cfg.layers[i].attention.pool for i in cfg.cache_users(j)} - {0}))


def build_pironex(cfg: PironexConfig, weights: WeightSet, ctx) -> ModelSpec:
    dt, dev = ctx.dtype, ctx.device
    eps, t = cfg.norm_eps, weights.take
    taps, n_layers = cfg.canon_taps, len(cfg.layers)
    embedding = Embedding(t("embed"), dt, dev, scale=cfg.embedding_scale)
    blocks, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        x = p + "mix."
        if layer.type == "attention":
            a = layer.attention
            own = a.kv_from is None
            owner = i if own else a.kv_from
            mixer = SoftmaxAttention(t(x + "q"), t(x + "k") if own else None, t(x + "v") if own else None, t(x + "o"), a.heads,
                                     a.kv_heads, a.dim, a.vdim, a.scale, window=a.window, rot_dims=a.rot_dims, rot_base=a.rot_base,
                                     softcap=a.softcap, shared_kv=not own, cache_keep=_cache_keep(cfg, owner), dtype=dt, device=dev,
                                     q_pre_norm=t(x + "q.norm"), k_pre_norm=t(x + "k.norm") if own else None, pre_norm_eps=eps,
                                     pool=a.pool, pooled_sizes=_pooled_sizes(cfg, owner))
            schedule.append(LayerCall(layer=i, cache=owner, write=own))
        elif layer.type == "mamba2":
            s = layer.ssm
            mixer = StateSpace(t(x + "in"), t(x + "conv"), t(x + "conv.b"), t(x + "dt_bias"), t(x + "A_log"), t(x + "D"), t(x + "norm"),
                               t(x + "o"), s.heads, s.vdim, s.state, s.groups, s.norm_groups, eps, dt, dev)
            schedule.append(LayerCall(layer=i, cache=None))
        else:
            c = layer.latent
            mixer = LatentAttention(t(x + "q"), t(x + "dkv"), t(x + "dkv.norm"), t(x + "uk"), t(x + "uv"), t(x + "o"), c.heads, c.dim,
                                    c.rot_dim, c.vdim, c.kv_rank, c.scale, c.rot_base, eps, dt, dev, window=c.window,
                                    pairing="interleaved")
            schedule.append(LayerCall(layer=i, cache=i))
        f = layer.mlp
        ff = pre2 = post2 = canon2 = None
        if f is not None:
            y = p + "mlp."
            shared = None
            if f.shared_ff:
                shared = (t(y + "shared.gate"), t(y + "shared.up"), t(y + "shared.down"), t(y + "shared.sg"), f.shared_limit)
            ff = RoutedExperts(t(y + "router"), [t(f"{y}e{e}.gate") for e in range(f.experts)],
                               [t(f"{y}e{e}.up") for e in range(f.experts)], [t(f"{y}e{e}.down") for e in range(f.experts)],
                               f.top, renormalize=True, dtype=dt, device=dev, activation="clamped_swish", limit=f.limit, shared=shared)
            pre2, post2 = LayerNorm(t(p + "norm2"), None, eps, dev), LayerNorm(t(p + "norm2b"), None, eps, dev)
            canon2 = t(p + "canon2") if taps else None
        blocks.append(SandwichBlock(LayerNorm(t(p + "norm1"), None, eps, dev), mixer, LayerNorm(t(p + "norm1b"), None, eps, dev),
                                    pre2, ff, post2, canon1=t(p + "canon1") if taps else None, canon2=canon2,
                                    depth_weights=t(p + "dwa"), depth_index=i, depth_slots=n_layers + 1, depth_name=DEPTH_STACK,
                                    device=dev))
    final_norm = LayerNorm(t("final.norm"), None, eps, dev)
    head = LMHead(embedding.table)                  # the embedding table itself, without its scale
    weights.finish()
    wbytes = sum(b.weight_bytes() for b in blocks) + final_norm.weight_bytes() + head.weight_bytes()
    return ModelSpec(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=final_norm, lm_head=head,
                     hidden_size=cfg.width, vocab_size=cfg.vocab, eos_token_ids=cfg.eos_token_ids, weight_bytes=wbytes,
                     step_buffers={DEPTH_STACK: ((n_layers + 1) * cfg.width, torch.float32)})


PIRONEX = Architecture(name=NAME, config_cls=PironexConfig, manifest=pironex_manifest, build=build_pironex)
register_architecture(PIRONEX, replace=True)
