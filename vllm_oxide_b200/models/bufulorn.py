"""The Bufulorn decoder as a list of parts.

embedding plus a learned vector per position; then the layers in order, each a `PostNormBlock` (the residual takes the
layer-normed result of each sub-layer; the sub-layers read the residual itself) whose mixer is a `SoftmaxAttention`
inside blocks of positions (biases, q and k normed per head with a shared weight, capped scores, a bias on the
logarithm of the distance, a sigmoid output gate; with `kv_from` it reads the cache of an earlier layer and has no key
and value tensors) or a `GatedDelta` with one decay per head and a silu gate, and whose feed-forward is an `ActMLP`
(xIELU), `RoutedExperts` or absent; then the model's layer norm and the head.

Tensor names are the checkpoint's own: `embed`, `pos`, `final.norm(.b)`, `head`, and per layer i `l<i>.norm1|norm2(.b)`,
`l<i>.mix.*` (`q k v` with `.b` biases, `q.norm k.norm r1 r2 g o`; or `q k v` with `.conv`, `b a A_log dt_bias g norm o`),
`l<i>.mlp.up|down|act` or `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`.
"""
from __future__ import annotations

from typing import Dict

from ..config.bufulorn_config import NAME, BufulornConfig
from ..config.registry import Architecture, register_architecture
from ..parts import Embedding, LayerCall, LMHead, ModelSpec
from ..parts.block import PostNormBlock
from ..parts.flex_attention import SoftmaxAttention
from ..parts.layernorm import LayerNorm
from ..parts.linear import to_compute
from ..parts.mlp import ActMLP
from ..parts.moe import RoutedExperts
from ..parts.recurrent import GatedDelta
from ..weights.loader import TensorSpec, WeightSet


def bufulorn_manifest(cfg: BufulornConfig) -> Dict[str, TensorSpec]:
    w = cfg.width
    m = {"embed": TensorSpec((cfg.vocab, w)), "pos": TensorSpec((cfg.max_positions, w))}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m[p + "norm1"], m[p + "norm1.b"] = TensorSpec((w,), init="ones"), TensorSpec((w,), init="zeros")
        x = p + "mix."
        if layer.type == "attention":
            a = layer.attention
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            m[x + "q"], m[x + "q.b"] = TensorSpec((nq, w)), TensorSpec((nq,))
            m[x + "q.norm"] = TensorSpec((a.dim,), init="ones")
            if a.kv_from is None:
                m[x + "k"], m[x + "k.b"] = TensorSpec((nk, w)), TensorSpec((nk,))
                m[x + "v"], m[x + "v.b"] = TensorSpec((nv, w)), TensorSpec((nv,))
                m[x + "k.norm"] = TensorSpec((a.dim,), init="ones")
            m[x + "r1"], m[x + "r2"] = TensorSpec((a.heads,), init="ones"), TensorSpec((a.heads,), init="ones")
            m[x + "g"] = TensorSpec((a.heads * a.vdim, w))
            m[x + "o"] = TensorSpec((w, a.heads * a.vdim))
        else:
            r = layer.delta
            gk, hv = r.kv_heads * r.dim, r.heads * r.vdim
            for n, rows in (("q", gk), ("k", gk), ("v", hv)):
                m[x + n] = TensorSpec((rows, w))
                m[x + n + ".conv"] = TensorSpec((rows, r.conv))
            m[x + "b"], m[x + "a"] = TensorSpec((r.heads, w)), TensorSpec((r.heads, w))
            m[x + "A_log"], m[x + "dt_bias"] = TensorSpec((r.heads,)), TensorSpec((r.heads,))
            m[x + "norm"] = TensorSpec((r.vdim,), init="ones")
            m[x + "g"] = TensorSpec((hv, w))
            m[x + "o"] = TensorSpec((w, hv))
        f = layer.mlp
        if f is not None:
            m[p + "norm2"], m[p + "norm2.b"] = TensorSpec((w,), init="ones"), TensorSpec((w,), init="zeros")
            y = p + "mlp."
            if f.kind == "dense":
                m[y + "up"], m[y + "down"], m[y + "act"] = TensorSpec((f.ff, w)), TensorSpec((w, f.ff)), TensorSpec((2,))
            else:
                m[y + "router"] = TensorSpec((f.experts, w))
                for e in range(f.experts):
                    m[f"{y}e{e}.gate"], m[f"{y}e{e}.up"] = TensorSpec((f.ff, w)), TensorSpec((f.ff, w))
                    m[f"{y}e{e}.down"] = TensorSpec((w, f.ff))
    m["final.norm"], m["final.norm.b"] = TensorSpec((w,), init="ones"), TensorSpec((w,), init="zeros")
    m["head"] = TensorSpec((cfg.vocab, w))
    return m


def _cache_keep(cfg: BufulornConfig, j: int):
    """What the cache that layer j writes must keep: its users' common block length, or everything when they differ
    (a block of one length is not made of whole blocks of another)."""
    sizes = {cfg.layers[i].attention.chunk for i in cfg.cache_users(j)}
    if len(sizes) == 1:
        size = sizes.pop()
        return ("chunk", size) if size else ("full", 0)
    return ("full", 0)


def build_bufulorn(cfg: BufulornConfig, weights: WeightSet, ctx) -> ModelSpec:
    dt, dev = ctx.dtype, ctx.device
    eps, t = cfg.norm_eps, weights.take
    embedding = Embedding(t("embed"), dt, dev, positions=t("pos"))
    blocks, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        x = p + "mix."
        if layer.type == "attention":
            a = layer.attention
            own = a.kv_from is None
            owner = i if own else a.kv_from
            mixer = SoftmaxAttention(t(x + "q"), t(x + "k") if own else None, t(x + "v") if own else None, t(x + "o"), a.heads,
                                     a.kv_heads, a.dim, a.vdim, a.scale, bias_q=t(x + "q.b"), bias_k=t(x + "k.b") if own else None,
                                     bias_v=t(x + "v.b") if own else None, unit_rms_eps=eps, q_norm_weight=t(x + "q.norm"),
                                     k_norm_weight=t(x + "k.norm") if own else None, chunk=a.chunk, softcap=a.softcap,
                                     dist_bias=(t(x + "r1"), t(x + "r2")), gate_weight=t(x + "g"), shared_kv=not own,
                                     cache_keep=_cache_keep(cfg, owner), dtype=dt, device=dev)
            schedule.append(LayerCall(layer=i, cache=owner, write=own))
        else:
            r = layer.delta
            mixer = GatedDelta(t(x + "q"), t(x + "k"), t(x + "v"), t(x + "q.conv"), t(x + "k.conv"), t(x + "v.conv"), t(x + "b"),
                               t(x + "A_log"), t(x + "a"), None, t(x + "dt_bias"), t(x + "g"), None, t(x + "norm"), t(x + "o"),
                               r.heads, r.kv_heads, r.dim, r.vdim, eps, dt, dev, gate="silu")
            schedule.append(LayerCall(layer=i, cache=None))
        norm1 = LayerNorm(t(p + "norm1"), t(p + "norm1.b"), eps, dev)
        f = layer.mlp
        if f is None:
            blocks.append(PostNormBlock(norm1, mixer, None, None))
            continue
        y = p + "mlp."
        if f.kind == "dense":
            ff = ActMLP(t(y + "up"), t(y + "down"), t(y + "act"), dt, dev, activation="xielu")
        else:
            ff = RoutedExperts(t(y + "router"), [t(f"{y}e{e}.gate") for e in range(f.experts)],
                               [t(f"{y}e{e}.up") for e in range(f.experts)], [t(f"{y}e{e}.down") for e in range(f.experts)],
                               f.top, f.groups, f.keep, renormalize=False, dtype=dt, device=dev)
        blocks.append(PostNormBlock(norm1, mixer, LayerNorm(t(p + "norm2"), t(p + "norm2.b"), eps, dev), ff))
    final_norm = LayerNorm(t("final.norm"), t("final.norm.b"), eps, dev)
    head = LMHead(to_compute(t("head"), dt, dev))
    weights.finish()
    wbytes = sum(b.weight_bytes() for b in blocks) + final_norm.weight_bytes() + head.weight_bytes()
    return ModelSpec(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=final_norm, lm_head=head,
                     hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_positions,
                     eos_token_ids=cfg.eos_token_ids, weight_bytes=wbytes)


BUFULORN = Architecture(name=NAME, config_cls=BufulornConfig, manifest=bufulorn_manifest, build=build_bufulorn)
register_architecture(BUFULORN, replace=True)
