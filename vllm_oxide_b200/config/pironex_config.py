"""Typed configuration of the Pironex decoder, read from config.json's own keys.

A Pironex model is a list of layers, each a norm on both sides of its mixer and of its feed-forward; what a sub-layer
reads first passes a short causal convolution over time that is added to it (`canon.taps`), and the stream that goes from
layer to layer is a learned weighted sum of the embedding's output and of every layer's result so far. A layer's mixer is
`attention` (a norm over the whole q and k projections, partial rotary positions, capped scores, a sliding window beside
which every block of `mask.pool` tokens that lies wholly before it counts as one pooled key and value; with `kv_from` the
layer reads an earlier layer's keys and values), `mamba2` (a selective state-space mixer) or `latent_attention` (attention
over a cached latent vector with a shared rotated key part, in a sliding window). The feed-forward is a mixture of small
experts with a clamped gate, beside a shared expert behind a sigmoid gate, or absent.

    {"architecture": "Pironex", "vocab": ..., "width": ..., "norm": {"eps": ...}, "embedding": {"scale": ...},
     "canon": {"taps": ...},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot": {"dims", "base"},
                           "mask": {"size", "pool"}, "kv_from": j},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"}}},
                {"type": "mamba2", "mixer": {"heads", "vdim", "state", "groups", "norm_groups", "conv"}, "mlp": ...},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}, "mask": {"size"}},
                 "mlp": null}]}

Every size and every constant that may differ between two models of the design is read here. Optional keys: `softcap`
(absent or 0: no cap), `rot` of an attention layer (absent: no rotation), `mask` (absent: every earlier token is seen),
`mask.pool` (absent or 0: nothing is seen behind the window), `kv_from`, `shared`, `mlp` (null: no feed-forward), `canon`
(absent: no convolution; one tap is still a convolution, without state), `embedding` (absent: scale 1).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from .lomopel_config import _heads
from .model_config import _need, _typed
from .rotepel_config import _obj

NAME = "Pironex"
LAYER_TYPES = ("attention", "mamba2", "latent_attention")


def _positive(where: str, **kw) -> None:
    for name, v in kw.items():
        if v <= 0:
            raise ConfigError(f"{where}: '{name}' must be positive")


@dataclass(frozen=True)
class PooledAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0                  # 0: scores are not capped
    rot_dims: int = 0                     # 0: no rotation
    rot_base: float = 10000.0
    window: int = 0                       # 0: every earlier token is seen
    pool: int = 0                         # 0: nothing is seen behind the window
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "PooledAttentionConfig":
        kw = _heads(m, where)
        kw["scale"] = _need(m, "scale", float, where)
        if m.get("softcap") is not None:
            kw["softcap"] = _typed(m, "softcap", float, where)
            if kw["softcap"] < 0:
                raise ConfigError(f"{where}: 'softcap' must not be negative")
        rot = _obj(m, "rot", where, optional=True)
        if rot is not None:
            kw["rot_dims"], kw["rot_base"] = _need(rot, "dims", int, where + ".rot"), _need(rot, "base", float, where + ".rot")
            if kw["rot_dims"] < 0 or kw["rot_dims"] % 2 or kw["rot_dims"] > kw["dim"] or kw["rot_base"] <= 0:
                raise ConfigError(f"{where}.rot: {kw['rot_dims']} rotated features (even, at most dim) with base {kw['rot_base']}")
        mask = _obj(m, "mask", where, optional=True)
        if mask is not None:
            kw["window"] = _need(mask, "size", int, where + ".mask")
            if mask.get("pool") is not None:
                kw["pool"] = _typed(mask, "pool", int, where + ".mask")
            if kw["window"] <= 0 or kw.get("pool", 0) < 0:
                raise ConfigError(f"{where}.mask: 'size' must be positive and 'pool' not negative")
        if m.get("kv_from") is not None:
            kw["kv_from"] = _typed(m, "kv_from", int, where)
        return cls(**kw)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.rot_dims:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        if self.window:
            d["mask"] = {"size": self.window, **({"pool": self.pool} if self.pool else {})}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "StateSpaceConfig":
        c = cls(**{k: _need(m, k, int, where) for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv")})
        _positive(where, heads=c.heads, vdim=c.vdim, state=c.state, groups=c.groups, norm_groups=c.norm_groups, conv=c.conv)
        if c.heads % c.groups or (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"{where}: {c.heads} heads of {c.vdim} do not split into {c.groups} groups and {c.norm_groups} norm groups")
        return c

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "norm_groups": self.norm_groups,
                "conv": self.conv}


@dataclass(frozen=True)
class WindowLatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    window: int = 0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "WindowLatentConfig":
        kw = {k: _need(m, k, int, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        _positive(where, **kw)
        kw["scale"] = _need(m, "scale", float, where)
        rot = _obj(m, "rot", where)
        kw["rot_base"] = _need(rot, "base", float, where + ".rot")
        if rot.get("dims") is not None and _typed(rot, "dims", int, where + ".rot") != kw["rot_dim"]:
            raise ConfigError(f"{where}.rot: 'dims' must equal 'rot_dim' ({kw['rot_dim']})")
        if kw["rot_dim"] % 2 or kw["rot_base"] <= 0:
            raise ConfigError(f"{where}: 'rot_dim' must be even and the base positive")
        mask = _obj(m, "mask", where, optional=True)
        if mask is not None:
            kw["window"] = _need(mask, "size", int, where + ".mask")
            if kw["window"] <= 0:
                raise ConfigError(f"{where}.mask: 'size' must be positive")
        return cls(**kw)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dim}}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class ClampedExpertsConfig:
    ff: int
    limit: float
    experts: int
    top: int
    shared_ff: int = 0                    # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "ClampedExpertsConfig":
        if m.get("kind") != "moe":
            raise ConfigError(f"{where}: kind {m.get('kind')!r} is not known (moe)")
        e, r = _obj(m, "expert", where), _obj(m, "router", where)
        kw = dict(ff=_need(e, "ff", int, where + ".expert"), limit=_need(e, "limit", float, where + ".expert"),
                  experts=_need(r, "experts", int, where + ".router"), top=_need(r, "top", int, where + ".router"))
        sh = _obj(m, "shared", where, optional=True)
        if sh is not None:
            kw["shared_ff"], kw["shared_limit"] = _need(sh, "ff", int, where + ".shared"), _need(sh, "limit", float, where + ".shared")
            if kw["shared_ff"] <= 0 or kw["shared_limit"] <= 0:
                raise ConfigError(f"{where}.shared: 'ff' and 'limit' must be positive")
        c = cls(**kw)
        if c.ff <= 0 or c.limit <= 0 or not 0 < c.top <= c.experts:
            raise ConfigError(f"{where}: {c.top} choices among {c.experts} experts of {c.ff} with limit {c.limit}")
        return c

    def to_dict(self) -> dict:
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class PironexLayer:
    type: str
    attention: Optional[PooledAttentionConfig] = None
    ssm: Optional[StateSpaceConfig] = None
    latent: Optional[WindowLatentConfig] = None
    mlp: Optional[ClampedExpertsConfig] = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PironexLayer":
        if not isinstance(d, dict):
            raise ConfigError(f"{where}: a layer must be an object")
        kind = d.get("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}: 'type' must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
        m = _obj(d, "mixer", where)
        kw = dict(type=kind)
        if kind == "attention":
            kw["attention"] = PooledAttentionConfig.from_dict(m, where + ".mixer")
        elif kind == "mamba2":
            kw["ssm"] = StateSpaceConfig.from_dict(m, where + ".mixer")
        else:
            kw["latent"] = WindowLatentConfig.from_dict(m, where + ".mixer")
        mlp = _obj(d, "mlp", where, optional=True)
        if mlp is not None:
            kw["mlp"] = ClampedExpertsConfig.from_dict(mlp, where + ".mlp")
        return cls(**kw)

    def to_dict(self) -> dict:
        m = self.attention or self.ssm or self.latent
        return {"type": self.type, "mixer": m.to_dict(), "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclass(frozen=True)
class PironexConfig:
    vocab: int
    width: int
    layers: Tuple[PironexLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    canon_taps: int = 0                   # 0: no convolution in front of the sub-layers
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "PironexConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        kw = dict(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                  layers=tuple(PironexLayer.from_dict(x, f"{where}: layers[{i}]") for i, x in enumerate(layers)),
                  norm_eps=_need(_obj(d, "norm", where), "eps", float, where + ".norm"))
        emb = _obj(d, "embedding", where, optional=True)
        if emb is not None and emb.get("scale") is not None:
            kw["embedding_scale"] = _typed(emb, "scale", float, where + ".embedding")
        canon = _obj(d, "canon", where, optional=True)
        if canon is not None:
            kw["canon_taps"] = _need(canon, "taps", int, where + ".canon")
            if kw["canon_taps"] < 1:
                raise ConfigError(f"{where}.canon: 'taps' must be at least 1")
        cfg = cls(**kw)
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{where}: vocab and width must be positive")
        for i, layer in enumerate(self.layers):
            a = layer.attention
            if a is None or a.kv_from is None:
                continue
            j = a.kv_from
            if not 0 <= j < i or self.layers[j].type != "attention" or self.layers[j].attention.kv_from is not None:
                raise ConfigError(f"{where}: layers[{i}].mixer.kv_from {j} must name an earlier attention layer with keys and "
                                  f"values of its own")
            b = self.layers[j].attention
            if (a.kv_heads, a.dim, a.vdim, a.rot_dims, a.rot_base) != (b.kv_heads, b.dim, b.vdim, b.rot_dims, b.rot_base):
                raise ConfigError(f"{where}: layers[{i}] reads the keys and values of layers[{j}] but its kv_heads, dim, vdim or "
                                  f"rotation differ")

    def cache_users(self, j: int) -> Tuple[int, ...]:
        """Layer j and the layers that read its keys and values."""
        return (j,) + tuple(i for i, x in enumerate(self.layers) if x.attention is not None and x.attention.kv_from == j)

    def param_count(self) -> int:
        from ..models.pironex import pironex_manifest
        total = 0
        for spec in pironex_manifest(self).values():
            n = 1
            for x in spec.shape:
                n *= max(int(x), 0)
            total += n
        return total

    def to_dict(self) -> dict:
        d = {"architecture": NAME, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "layers": [x.to_dict() for x in self.layers]}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        return d
