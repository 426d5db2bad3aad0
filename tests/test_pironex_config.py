"""The Pironex configuration on the CPU: config.json's keys in and out, optional keys, what is refused, which cache a layer
that reads another's keys and values needs, the manifest of tensor names, model folders with random weights."""
import json
import os

import pytest
import torch

from vllm_oxide_b200.config import ClampedExpertsConfig, PironexConfig, architecture_for
from vllm_oxide_b200.errors import ConfigError
from vllm_oxide_b200 import models  # noqa: F401  (registers the architectures)


def _dict():
    moe = {"kind": "moe", "expert": {"ff": 24, "limit": 1.0}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 40, "limit": 2.5}}
    return {"architecture": "Pironex", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 6.0}, "canon": {"taps": 3},
            "layers": [
                {"type": "mamba2", "mixer": {"heads": 4, "vdim": 16, "state": 8, "groups": 2, "norm_groups": 1, "conv": 3}, "mlp": moe},
                {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.2, "softcap": 6.0,
                                                "rot": {"dims": 8, "base": 100.0}, "mask": {"size": 10, "pool": 4}}, "mlp": moe},
                {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 32, "scale": 0.2,
                                                       "rot": {"base": 1000.0, "dims": 8}, "mask": {"size": 13}}, "mlp": None},
                {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3,
                                                "rot": {"dims": 8, "base": 100.0}, "mask": {"size": 7}, "kv_from": 1}, "mlp": None}]}


def test_keys_in_and_out_and_the_registry():
    d = _dict()
    cfg = PironexConfig.from_dict(d)
    assert cfg.to_dict() == d
    assert PironexConfig.from_dict(cfg.to_dict()) == cfg
    assert architecture_for(d).name == "Pironex"
    a, r = cfg.layers[1].attention, cfg.layers[3].attention
    assert (a.window, a.pool, a.softcap, a.rot_dims, a.kv_from) == (10, 4, 6.0, 8, None)
    assert (r.window, r.pool, r.softcap, r.kv_from) == (7, 0, 0.0, 1)
    assert cfg.layers[2].latent.window == 13 and cfg.layers[2].mlp is None
    assert cfg.layers[0].mlp == ClampedExpertsConfig(ff=24, limit=1.0, experts=6, top=2, shared_ff=40, shared_limit=2.5)
    assert cfg.cache_users(1) == (1, 3)


def test_optional_keys_switch_their_mechanism_off():
    d = _dict()
    del d["canon"], d["embedding"]
    d["layers"][1]["mixer"].pop("mask")
    d["layers"][1]["mixer"].pop("rot")
    d["layers"][3]["mixer"].pop("rot")
    d["layers"][2]["mixer"].pop("mask")
    d["layers"][0]["mlp"] = dict(d["layers"][0]["mlp"])
    d["layers"][0]["mlp"].pop("shared")
    cfg = PironexConfig.from_dict(d)
    assert cfg.canon_taps == 0 and cfg.embedding_scale == 1.0
    assert cfg.layers[1].attention.window == 0 and cfg.layers[1].attention.rot_dims == 0 and cfg.layers[2].latent.window == 0
    assert cfg.layers[0].mlp.shared_ff == 0
    assert "canon" not in cfg.to_dict()


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(dim=32), "differ"),
    (lambda d: d["layers"][3]["mixer"]["rot"].update(base=7.0), "differ"),
    (lambda d: d["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "rot"),
    (lambda d: d["layers"][0]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "choices"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["canon"].update(taps=0), "taps"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_what_is_refused(change, word):
    d = json.loads(json.dumps(_dict()))
    change(d)
    with pytest.raises(ConfigError) as e:
        PironexConfig.from_dict(d)
    assert word in str(e.value)


def test_manifest_names_and_a_model_folder(tmp_path):
    from vllm_oxide_b200.config.model_config import write_config_json
    from vllm_oxide_b200.models import pironex_manifest
    from vllm_oxide_b200.weights import load_safetensors_weights, random_tensors
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    cfg = PironexConfig.from_dict(_dict())
    m = pironex_manifest(cfg)
    assert m["l0.mix.in"].shape == (2 * 64 + 2 * 16 + 4, 64) and m["l0.mix.conv"].shape == (64 + 32, 3)
    assert m["l1.mix.q.norm"].shape == (96,) and m["l1.mix.k.norm"].shape == (48,)
    assert "l3.mix.k" not in m and "l3.mix.k.norm" not in m and "l3.mix.v" not in m          # it reads layer 1's
    assert "l2.norm2" not in m and "l2.canon2" not in m and "l2.mlp.router" not in m         # no feed-forward
    assert m["l2.mix.dkv"].shape == (40, 64) and m["l0.mlp.shared.sg"].shape == (1, 64)
    assert [m[f"l{i}.dwa"].shape for i in range(4)] == [(2,), (3,), (4,), (5,)]
    assert "head" not in m and m["final.norm"].shape == (64,)
    assert cfg.param_count() == sum(int(torch.tensor(s.shape).prod()) for s in m.values())
    d = str(tmp_path)
    write_config_json(d, cfg.to_dict())
    write_safetensors(os.path.join(d, "model.safetensors"), random_tensors(m, 5, 0.1, torch.bfloat16, "cpu"))
    w = load_safetensors_weights(d, m, device="cpu")
    assert w.take("l1.canon1").shape == (64, 3)
