"""Typed configuration of the Bufulorn decoder, read from config.json's own keys.

A Bufulorn model is a list of layers; the residual takes the layer-normed result of each sub-layer, and the sub-layers
read the residual itself. A layer of type `attention` has softmax attention inside blocks of positions (biased
projections, q and k normed per head with a shared weight, capped scores, a bias that grows with the logarithm of the
distance, a sigmoid output gate) and may take its keys and values from an earlier layer's cache (`kv_from`); a layer
of type `delta` has a gated delta rule with short causal convolutions and one decay per head. A layer's feed-forward
is dense (not gated, xIELU), a mixture of small gated experts chosen among the best groups, or absent. A learned
vector per position is added to the embedding.

    {"architecture": "Bufulorn", "vocab": ..., "width": ..., "max_positions": ..., "norm": {"eps": ...},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask": {"size"}, "kv_from": j},
                 "mlp": {"kind": "dense", "ff": ...}},
                {"type": "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"},
                 "mlp": {"kind": "moe", "expert": {"ff": ...},
                         "router": {"experts": ..., "top": ..., "groups": {"count": ..., "keep": ...}}}}]}

Every size and every constant that may differ between two models of the design is read here. Optional keys: `mask`
(absent: every earlier token is seen), `softcap` (absent or 0: scores are not capped), `kv_from` (absent: the layer has
keys and values of its own), `groups` (absent: every expert stands for election), `mlp` (null: no feed-forward).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from .lomopel_config import _heads
from .model_config import _need, _typed
from .rotepel_config import _obj

NAME = "Bufulorn"
LAYER_TYPES = ("attention", "delta")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class ChunkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0                  # 0: scores are not capped
    chunk: int = 0                        # length of a block of positions; 0: all earlier tokens are seen
    kv_from: Optional[int] = None         # the layer whose cached keys and values this one reads

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "ChunkAttentionConfig":
        kw = _heads(m, where)
        kw["scale"] = _need(m, "scale", float, where)
        if m.get("softcap") is not None:
            kw["softcap"] = _typed(m, "softcap", float, where)
            if kw["softcap"] < 0:
                raise ConfigError(f"{where}: 'softcap' must not be negative")
        mask = _obj(m, "mask", where, optional=True)
        if mask is not None:
            kw["chunk"] = _need(mask, "size", int, where + ".mask")
            if kw["chunk"] <= 0:
                raise ConfigError(f"{where}.mask: 'size' must be positive")
        if m.get("kv_from") is not None:
            kw["kv_from"] = _typed(m, "kv_from", int, where)
        return cls(**kw)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class HeadDecayDeltaConfig:
    """The gated delta rule with one decay per head and full projections for the decay and the gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "HeadDecayDeltaConfig":
        kw = _heads(m, where)
        kw["conv"] = _need(m, "conv", int, where)
        if kw["conv"] < 1:
            raise ConfigError(f"{where}: 'conv' must be at least 1")
        return cls(**kw)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                             # "dense" or "moe"
    ff: int                               # hidden size of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    groups: int = 0                       # 0: no groups
    keep: int = 0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "FeedForwardConfig":
        kind = m.get("kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"{where}: kind {kind!r} is not known ({', '.join(MLP_KINDS)})")
        if kind == "dense":
            kw = dict(kind=kind, ff=_need(m, "ff", int, where))
        else:
            r = _obj(m, "router", where)
            kw = dict(kind=kind, ff=_need(_obj(m, "expert", where), "ff", int, where + ".expert"),
                      experts=_need(r, "experts", int, where + ".router"), top=_need(r, "top", int, where + ".router"))
            g = _obj(r, "groups", where + ".router", optional=True)
            if g is not None:
                kw["groups"] = _need(g, "count", int, where + ".router.groups")
                kw["keep"] = _need(g, "keep", int, where + ".router.groups")
        cfg = cls(**kw)
        if cfg.ff <= 0:
            raise ConfigError(f"{where}: 'ff' must be positive")
        if kind == "moe":
            if not 0 < cfg.top <= cfg.experts:
                raise ConfigError(f"{where}.router: {cfg.top} choices among {cfg.experts} experts")
            if cfg.groups and (cfg.groups < 0 or cfg.experts % cfg.groups or not 0 < cfg.keep <= cfg.groups
                               or cfg.top > cfg.keep * (cfg.experts // cfg.groups)):
                raise ConfigError(f"{where}.router: {cfg.experts} experts in {cfg.groups} groups of which {cfg.keep} are kept "
                                  f"cannot give {cfg.top} choices")
        return cfg

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        r = {"experts": self.experts, "top": self.top}
        if self.groups:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": r}


@dataclass(frozen=True)
class BufulornLayer:
    type: str
    attention: Optional[ChunkAttentionConfig] = None     # type "attention"
    delta: Optional[HeadDecayDeltaConfig] = None          # type "delta"
    mlp: Optional[FeedForwardConfig] = None               # None: the layer has no feed-forward

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "BufulornLayer":
        if not isinstance(d, dict):
            raise ConfigError(f"{where}: a layer must be an object")
        kind = d.get("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}: 'type' must be one of {', '.join(LAYER_TYPES)}, got {kind!r}")
        m = _obj(d, "mixer", where)
        kw = dict(type=kind)
        if kind == "attention":
            kw["attention"] = ChunkAttentionConfig.from_dict(m, where + ".mixer")
        else:
            kw["delta"] = HeadDecayDeltaConfig.from_dict(m, where + ".mixer")
        mlp = _obj(d, "mlp", where, optional=True)
        if mlp is not None:
            kw["mlp"] = FeedForwardConfig.from_dict(mlp, where + ".mlp")
        return cls(**kw)

    def to_dict(self) -> dict:
        m = self.attention.to_dict() if self.type == "attention" else self.delta.to_dict()
        return {"type": self.type, "mixer": m, "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclass(frozen=True)
class BufulornConfig:
    vocab: int
    width: int
    layers: Tuple[BufulornLayer, ...]
    norm_eps: float
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "BufulornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        norm = _obj(d, "norm", where)
        cfg = cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                  layers=tuple(BufulornLayer.from_dict(x, f"{where}: layers[{i}]") for i, x in enumerate(layers)),
                  norm_eps=_need(norm, "eps", float, where + ".norm"), max_positions=_need(d, "max_positions", int, where))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0:
            raise ConfigError(f"{where}: vocab, width and max_positions must be positive")
        for i, layer in enumerate(self.layers):
            a = layer.attention
            if a is None or a.kv_from is None:
                continue
            j = a.kv_from
            if not 0 <= j < i or self.layers[j].type != "attention" or self.layers[j].attention.kv_from is not None:
                raise ConfigError(f"{where}: layers[{i}].mixer.kv_from {j} must name an earlier attention layer with keys and "
                                  f"values of its own")
            b = self.layers[j].attention
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"{where}: layers[{i}] reads the keys and values of layers[{j}] but its kv_heads, dim or vdim "
                                  f"differ")

    def cache_users(self, j: int) -> Tuple[int, ...]:
        """Layer j and the layers that read its keys and values."""
        return (j,) + tuple(i for i, x in enumerate(self.layers) if x.attention is not None and x.attention.kv_from == j)

    def param_count(self) -> int:
        from ..models.bufulorn import bufulorn_manifest
        total = 0
        for spec in bufulorn_manifest(self).values():
            n = 1
            for x in spec.shape:
                n *= max(int(x), 0)
            total += n
        return total

    def to_dict(self) -> dict:
        return {"architecture": NAME, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "norm": {"eps": self.norm_eps}, "layers": [x.to_dict() for x in self.layers]}
