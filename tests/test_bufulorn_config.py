"""The Bufulorn configuration: config.json's keys in, the same keys out; optional keys; what is refused; the manifest
that follows from it; what the shared caches must keep; random model folders; the chunk kind of cache group (CPU only)."""
import json
import os

import pytest
import torch

from vllm_oxide_b200 import models  # noqa: F401  (registers the architectures)
from vllm_oxide_b200.config import BufulornConfig, architecture_for
from vllm_oxide_b200.errors import ConfigError, WeightsError
from vllm_oxide_b200.models import bufulorn_manifest


def _dict():
    def att(**more):
        return dict({"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "softcap": 30.0, "mask": {"size": 11}}, **more)
    moe = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 3}}}
    return {
        "architecture": "Bufulorn", "vocab": 90, "width": 40, "max_positions": 128, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "attention", "mixer": att(), "mlp": {"kind": "dense", "ff": 64}},
            {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}, "mlp": moe},
            {"type": "attention", "mixer": att(heads=6, kv_from=0), "mlp": None},
        ]}


def test_keys_in_keys_out_and_the_registry():
    d = _dict()
    arch = architecture_for(d)
    assert arch.name == "Bufulorn"
    cfg = arch.config_cls.from_dict(d)
    assert isinstance(cfg, BufulornConfig)
    assert cfg.to_dict() == d
    assert BufulornConfig.from_dict(cfg.to_dict()) == cfg
    a, r, f = cfg.layers[0].attention, cfg.layers[1].delta, cfg.layers[1].mlp
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, a.chunk, a.kv_from) == (4, 2, 12, 20, 0.3, 30.0, 11, None)
    assert (r.heads, r.kv_heads, r.dim, r.vdim, r.conv) == (4, 2, 8, 12, 3)
    assert (f.kind, f.ff, f.experts, f.top, f.groups, f.keep) == ("moe", 24, 8, 2, 4, 3)
    assert cfg.layers[2].attention.kv_from == 0 and cfg.layers[2].mlp is None and cfg.layers[0].mlp.ff == 64
    assert cfg.cache_users(0) == (0, 2) and cfg.max_positions == 128 and cfg.norm_eps == 1e-6
    assert cfg.param_count() == sum(torch.Size(s.shape).numel() for s in bufulorn_manifest(cfg).values())


def test_optional_keys():
    d = _dict()
    del d["layers"][0]["mixer"]["softcap"]
    del d["layers"][0]["mixer"]["mask"]
    del d["layers"][1]["mlp"]["router"]["groups"]
    cfg = BufulornConfig.from_dict(d)
    assert cfg.layers[0].attention.softcap == 0.0 and cfg.layers[0].attention.chunk == 0 and cfg.layers[1].mlp.groups == 0
    assert cfg.to_dict() == d


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "parallel"), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "mask", "size"), 0),
    (("layers", 0, "mixer", "softcap"), -1.0), (("layers", 1, "mixer", "conv"), 0), (("layers", 0, "mlp", "kind"), "gated"),
    (("layers", 2, "mixer", "kv_from"), 1), (("layers", 2, "mixer", "kv_from"), 2), (("layers", 2, "mixer", "vdim"), 16),
    (("layers", 0, "mixer", "kv_from"), 0), (("layers", 1, "mlp", "router", "top"), 9), (("layers", 1, "mlp", "router", "groups", "count"), 3),
    (("layers", 1, "mlp", "router", "groups", "keep"), 5), (("layers", 1, "mlp", "router", "top"), 7), (("layers", 0, "mixer", "scale"), "big"),
    (("max_positions",), 0), (("norm",), None), (("layers",), [])])
def test_what_is_refused(path, value):
    d = _dict()
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        BufulornConfig.from_dict(d)


def test_manifest_names_and_shapes():
    m = bufulorn_manifest(BufulornConfig.from_dict(_dict()))
    assert m["embed"].shape == (90, 40) and m["pos"].shape == (128, 40) and m["head"].shape == (90, 40)
    assert m["final.norm"].shape == (40,) and m["final.norm.b"].shape == (40,)
    assert m["l0.mix.q"].shape == (48, 40) and m["l0.mix.q.b"].shape == (48,) and m["l0.mix.k"].shape == (24, 40)
    assert m["l0.mix.v"].shape == (40, 40) and m["l0.mix.v.b"].shape == (40,) and m["l0.mix.o"].shape == (40, 80)
    assert m["l0.mix.q.norm"].shape == (12,) and m["l0.mix.k.norm"].shape == (12,) and m["l0.mix.r1"].shape == (4,)
    assert m["l0.mix.g"].shape == (80, 40) and "l0.mix.o.b" not in m
    assert m["l0.mlp.up"].shape == (64, 40) and m["l0.mlp.down"].shape == (40, 64) and m["l0.mlp.act"].shape == (2,)
    assert m["l1.mix.q"].shape == (16, 40) and m["l1.mix.q.conv"].shape == (16, 3) and m["l1.mix.v.conv"].shape == (48, 3)
    assert m["l1.mix.b"].shape == (4, 40) and m["l1.mix.a"].shape == (4, 40) and m["l1.mix.dt_bias"].shape == (4,)
    assert m["l1.mix.g"].shape == (48, 40) and m["l1.mix.norm"].shape == (12,) and m["l1.mix.o"].shape == (40, 48)
    assert m["l1.mlp.router"].shape == (8, 40) and m["l1.mlp.e7.gate"].shape == (24, 40) and m["l1.mlp.e0.down"].shape == (40, 24)
    assert "l1.mlp.e8.up" not in m and m["l1.norm2.b"].shape == (40,)
    # the layer that reads another layer's keys and values has none of their tensors, and without feed-forward no second norm
    assert m["l2.mix.q"].shape == (72, 40) and m["l2.mix.r2"].shape == (6,) and m["l2.mix.q.norm"].shape == (12,)
    for name in ("l2.mix.k", "l2.mix.k.b", "l2.mix.v", "l2.mix.k.norm", "l2.norm2", "l2.mlp.up"):
        assert name not in m


def test_what_a_shared_cache_keeps():
    """Users with one block length: the cache keeps the current block; with different ones (or one that sees
    everything): it keeps everything."""
    from vllm_oxide_b200.models.bufulorn import _cache_keep
    d = _dict()
    assert _cache_keep(BufulornConfig.from_dict(d), 0) == ("chunk", 11)
    d["layers"][2]["mixer"]["mask"]["size"] = 22
    assert _cache_keep(BufulornConfig.from_dict(d), 0) == ("full", 0)
    del d["layers"][2]["mixer"]["mask"]
    assert _cache_keep(BufulornConfig.from_dict(d), 0) == ("full", 0)
    del d["layers"][0]["mixer"]["mask"]
    assert _cache_keep(BufulornConfig.from_dict(d), 0) == ("full", 0)


def test_a_random_model_folder_reads_back_and_a_wrong_one_is_refused(tmp_path):
    from vllm_oxide_b200.weights import load_safetensors_weights, write_random_model
    from vllm_oxide_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = BufulornConfig.from_dict(_dict())
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=3, std=0.1)
    assert json.load(open(os.path.join(d, "config.json"))) == _dict()
    manifest = bufulorn_manifest(cfg)
    ws = load_safetensors_weights(d, manifest)
    assert ws.take("l1.mlp.e3.up").shape == (24, 40) and not ws.has("l2.mix.k")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["l2.mix.k"] = torch.zeros(24, 40, dtype=torch.bfloat16)
    del tensors["l0.mix.r1"]
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_safetensors_weights(d, manifest)
    assert e.value.missing == ["l0.mix.r1"] and e.value.unexpected == ["l2.mix.k"]


def test_chunk_groups_give_back_the_pages_behind_the_current_block():
    """Blocks of 20 positions over pages of 8: a query at position p reads from p - p % 20 on; a page goes back as soon
    as the next query's block starts behind it, also in the middle of a page, and is handed out again."""
    from vllm_oxide_b200.csrc.build import runtime_module
    rt = runtime_module()
    m = rt.CacheManager(8, [rt.GroupSpec(rt.CHUNK, 20, 6)], 2)
    assert [m.first_visible(0, p) for p in (0, 19, 20, 39, 40, 59)] == [0, 0, 20, 20, 40, 40]
    assert m.max_pages_held(0, 1000) == 4              # a block of 20 and the page it starts inside: 28 tokens
    assert m.admit(1) >= 0
    assert m.reserve(1, 19) and not m.commit(1, 19)    # positions 0..18: pages 0..2 held, the next query still in block 0
    held = list(m.block_table(1, 0))
    assert len(held) == 3 and all(p >= 0 for p in held)
    assert m.reserve(1, 1)
    released = m.commit(1, 1)                          # the next query sits at 20: pages 0 and 1 (positions 0..15) are behind
    assert sorted(p for _, p in released) == sorted(held[:2])
    assert list(m.block_table(1, 0))[:2] == [-1, -1] and m.slot_of(1, 0, 19) == held[2] * 8 + 3
    assert m.reserve(1, 27) and m.commit(1, 27) != []  # on to position 47: the block from 40 on is what is left
    table = list(m.block_table(1, 0))
    assert table[:5] == [-1] * 5 and table[5] >= 0 and m.check_invariants() == ""
    m.release(1)
    assert m.num_free_pages(0) == 6 and m.check_invariants() == ""
