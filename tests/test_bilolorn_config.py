"""Bilolorn's configuration and spec, and the cache bookkeeping it relies on; no device needed."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_bilolorn as plain
from cuinfer_b200.cache import CacheGroupSpec, CacheManager, group_runs, page_bytes
from cuinfer_b200.config import ConfigError, architecture_of
from cuinfer_b200.models.bilolorn import BilolornConfig, bilolorn_spec, run_order
from cuinfer_b200.parts import DecoderModel, PagedCacheNeed
from cuinfer_b200.weights.random_init import random_tensors


def _cfg(loop=(1, 3, 2)):
    mixer = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.25, "rot": {"base": 100.0, "dims": 4}}
    layers = [{"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": 20}},
              {"type": "latent_attention", "mixer": dict(mixer, heads=3), "mlp": None},
              {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 8},
                                                                     "shared": {"ff": 6}}},
              {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 8}}}]
    return {"architecture": "Bilolorn", "vocab": 50, "width": 16, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5}, "layers": layers,
            "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}}


def test_the_architecture_is_found_by_either_key():
    raw = _cfg()
    assert architecture_of(raw).name == "Bilolorn"
    assert architecture_of({"architectures": ["Bilolorn"]}).name == "Bilolorn"
    with pytest.raises(ConfigError):
        architecture_of({"architecture": ""})


@pytest.mark.parametrize("loop, order, again", [((1, 3, 2), (0, 1, 2, 1, 2, 3), (3,)), ((0, 4, 3), tuple(range(4)) * 3, (4, 8)),
                                               ((2, 2, 5), (0, 1, 2, 3), ()), ((0, 1, 1), (0, 1, 2, 3), ()), ((3, 4, 2), (0, 1, 2, 3, 3), (4,))])
def test_run_order_matches_the_plain_one(loop, order, again):
    cfg = BilolornConfig.from_dict(_cfg(loop))
    assert run_order(cfg) == (order, again)
    runs = plain.run_order(_cfg(loop))
    assert tuple(l for l, _ in runs) == order and tuple(i for i, (_, a) in enumerate(runs) if a) == again
    spec = bilolorn_spec(cfg)
    assert spec.run_order() == order and spec.reinject_embedding_before == again and spec.embedding_scale == 1.5


def test_spec_names_every_tensor_once_and_each_run_has_a_cache():
    cfg = BilolornConfig.from_dict(_cfg())
    model = DecoderModel(bilolorn_spec(cfg), torch.float32)
    names = [t.name for t in model.tensors()]
    assert len(names) == len(set(names))
    assert "l1.norm2" not in names and "l1.norm1b.b" in names and "l2.mlp.shared.up" in names and "l3.mlp.shared.up" not in names
    assert "l2.mlp.e3.down" in names and "l3.mlp.e2.gate" in names and "l3.mlp.e3.gate" not in names
    by_name = {t.name: t for t in model.tensors()}
    assert by_name["l2.mlp.table"].integer and by_name["l2.mlp.table"].shape == (50, 2) and by_name["l1.mix.g"].shape == (18, 16)
    needs = model.cache_needs()
    assert sorted(needs) == list(range(6)) and all(n == PagedCacheNeed(1, 16, None, planes=1) for n in needs.values())
    groups = group_runs(needs)
    assert len(groups) == 1 and groups[0].planes == 1 and page_bytes(groups[0], 16, torch.float32) == 6 * 16 * 16 * 4
    assert model.capturable


def test_random_weights_fit_the_plain_implementation():
    raw = _cfg()
    tensors = random_tensors(raw, seed=4, std=0.2, gain_std=0.1)
    table = tensors["l2.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 4 and bool((table[:, 0] != table[:, 1]).all())
    assert float(tensors["l0.norm1.b"].abs().max()) > 0 and abs(float(tensors["l0.norm1"].mean()) - 1) < 0.2
    logits = plain.forward(raw, {k: (v if v.dtype == torch.int32 else v.double()) for k, v in tensors.items()}, [3, 1, 4, 1, 5])
    assert logits.shape == (5, 50) and bool(torch.isfinite(logits).all())


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"), (lambda c: c["layers"][0]["mixer"].update(heads=0), "positive"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"), (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["loop"].update(stop=9), "loop"), (lambda c: c["loop"].update(times=0), "loop"), (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=5), "top"), (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c.update(layers=[]), "layers"), (lambda c: c["embedding"].pop("scale"), "scale")])
def test_bad_configurations_are_refused(change, word):
    raw = copy.deepcopy(_cfg())
    change(raw)
    with pytest.raises(ConfigError, match=word):
        BilolornConfig.from_dict(raw)


def test_config_round_trip():
    cfg = BilolornConfig.from_dict(_cfg())
    assert BilolornConfig.from_dict(cfg.to_dict()) == cfg


def test_one_plane_groups_are_kept_apart_from_two_plane_ones():
    needs = {0: PagedCacheNeed(1, 16, None, planes=1), 1: PagedCacheNeed(1, 16), 2: PagedCacheNeed(1, 16, None, planes=1)}
    groups = group_runs(needs)
    assert sorted((g.runs, g.planes) for g in groups) == [((0, 2), 1), ((1,), 2)]
    mgr = CacheManager(groups, 4, 6, 2)
    assert mgr.admit("a") == 0 and mgr.allocate("a", 9) and [len(mgr.block_table("a", g)) for g in range(2)] == [3, 3]
    mgr.commit("a", 9)
    mgr.release("a")
    assert mgr.admit("b") == 0 and mgr.allocate("b", 24)
    mgr.commit("b", 24)
    assert not mgr.allocate("b", 1)
    mgr.check()
