"""Kusolorn's configuration reader and its model written down as data (no GPU): tensor names and shapes, which
attention layer publishes its values and which mix them in, cache groups with kept first tokens, refusals, and the
page bookkeeping of a window that keeps the first tokens."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_kusolorn as plain
from cuinfer_b200.cache import CacheManager, group_runs
from cuinfer_b200.config.model_config import ConfigError
from cuinfer_b200.config.registry import architecture_of
from cuinfer_b200.parts import DecoderModel


def attention(heads=4, kv_heads=2, dim=16, vdim=8, window=12, keep=3, v_mix=True, rot=8, softcap=20.0, scaling=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.4, "softcap": softcap, "v_mix": v_mix}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot:
        m["rot"] = {"base": 1000.0, "dims": rot}
        if scaling:
            m["rot"]["scaling"] = {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 64}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": 40}}


MOE = {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 24, "limit": 1.5}}
CFG = {"architecture": "Kusolorn", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "token_side": {"dim": 6}, "layers": [
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 12, "vdim": 20, "gate_cap": 10.0}, "mlp": MOE},
    attention(v_mix=False, window=None),
    attention(),
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}, "mlp": None},
    attention(window=20, keep=0, softcap=None, scaling=False),
]}


def _build(cfg):
    arch = architecture_of(cfg)
    typed = arch.parse(cfg)
    return typed, arch.spec(typed), DecoderModel(arch.spec(typed), torch.float32)


def test_tensor_names_and_shapes_are_those_of_the_plain_model():
    _typed, _spec, model = _build(CFG)
    want = {k: tuple(v.shape) for k, v in plain.random_model(CFG, 0).items()}
    got = {t.name: tuple(t.shape) for t in model.tensors()}
    assert got == want


def test_roles_of_value_mixing_and_what_layers_keep():
    typed, spec, model = _build(CFG)
    roles = [l.mixer.get("value_mix") for l in spec.layers]
    assert roles == [None, None, "source", None, "mixed"]
    needs = model.cache_needs()
    assert sorted(needs) == [1, 2, 4]
    assert (needs[1].window, needs[1].keep_first, needs[1].planes, needs[1].head_dim) == (None, 0, 1, 24)
    assert (needs[2].window, needs[2].keep_first) == (12, 3) and (needs[4].window, needs[4].keep_first) == (20, 0)
    assert len(group_runs(needs)) == 3
    states = model.state_needs()
    assert states[0].shape == (2, 12 * 20 + 12 + 1)
    assert {s.name: s.shape for s in states[3]} == {"memory": (4, 8 * 12), "conv": (2, 2 * 2 * 8 + 4 * 12)}
    assert typed.to_dict()["layers"][2]["mixer"]["mask"] == {"size": 12, "keep_first": 3}
    assert architecture_of(typed.to_dict()).parse(typed.to_dict()) == typed
    assert model.capturable


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "rwkv", "type"),
    (("layers", 2, "mixer", "heads"), 3, "multiple of kv_heads"),
    (("layers", 2, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mlp", "router", "top"), 9, "exceeds"),
    (("layers", 0, "mlp", "kind"), "glu", "dense or moe"),
    (("layers", 3, "mixer", "conv"), 0, "positive"),
    (("layers", 4, "mixer", "vdim"), 16, "agree"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_refusals(path, value, message):
    cfg = copy.deepcopy(CFG)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).parse(cfg)


def test_scaled_frequencies_follow_the_plain_rule():
    from cuinfer_b200.parts.position import RotaryInterleaved
    from cuinfer_b200.parts.spec import PartSpec

    for dims, base, scaling in ((8, 1000.0, (6.0, 1.0, 3.0, 64)), (32, 2e5, (8.0, 2.0, 6.0, 512)), (6, 50.0, None)):
        part = RotaryInterleaved(PartSpec("rope_interleaved", theta=base, rotary_dim=dims, scaling=scaling), hidden_size=8,
                                 prefix="x", dtype=torch.float32)
        raw = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
        want = torch.tensor(plain.rotary_frequencies(base, dims, raw), dtype=torch.float64)
        assert torch.allclose(part.host_frequencies().double(), want, rtol=1e-6, atol=0)
    kinds = {round(f / (1000.0 ** (-2.0 * i / 8)), 6) for i, f in enumerate(plain.rotary_frequencies(1000.0, 8, {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 64}))}
    assert 1.0 in kinds and round(1 / 6, 6) in kinds and len(kinds) >= 3, "the test's constants must reach all three branches"


def test_pages_behind_a_window_are_given_back_except_those_of_the_kept_tokens():
    needs = _build(CFG)[2].cache_needs()
    groups = group_runs(needs)
    page = 4
    mgr = CacheManager(groups, page, 64, 2)
    kept = next(i for i, g in enumerate(groups) if g.keep_first == 3)
    plain_window = next(i for i, g in enumerate(groups) if g.window == 20)
    everything = next(i for i, g in enumerate(groups) if g.window is None)
    mgr.admit("a")
    total = 0
    for n in (5, 2, 30, 1, 1, 9):
        assert mgr.allocate("a", n)
        mgr.commit("a", n)
        total += n
        for g, window, keep in ((kept, 12, 3), (plain_window, 20, 0), (everything, None, 0)):
            table = mgr.block_table("a", g)
            for idx, p in enumerate(table):
                first, last = idx * page, idx * page + page - 1
                needed = window is None or last >= total - window + 1 or first < keep      # by the next query, at ``total``
                assert (p >= 0) == needed, f"group {g}: page {idx} after {total} tokens"
        mgr.check()
    mgr.release("a")
    assert all(pool.num_free == 64 for pool in mgr.pools)
