"""The Norelix design's host side on the CPU: configuration, tensor names, cache needs, the layer order with shared
keys and values, page release under a window that keeps a request's first keys, and the plain implementation's own
mechanisms against closed forms.  (What runs kernels is in test_norelix_gpu.py.)"""
from __future__ import annotations

import copy
import json

import numpy as np
import pytest
import torch

import plain_norelix as pn
from swifttransformer_b200.cache.manager import CacheManager, PagedCacheView, StateView
from swifttransformer_b200.config import ConfigError, NorelixConfig, load_config
from swifttransformer_b200.models import build_model_def, write_random_model
from swifttransformer_b200.parts.base import PagedKVSpec, StateSpec


def raw_config():
    left = dict(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.3, mask={"size": 20, "keep_first": 6},
                rot={"dims": 4, "base": 100.0})
    right = dict(heads=4, kv_heads=2, dim=6, vdim=10, conv=3)
    par = {"type": "parallel", "mlp": {"kind": "dense", "ff": 40, "limit": 2.5},
           "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 1.2}}
    att = {"type": "attention", "mlp": None,
           "mixer": dict(heads=6, kv_heads=3, dim=10, vdim=14, scale=0.2, q_temp={"coef": 0.3, "every": 5})}
    shared = {"type": "attention", "mlp": {"kind": "dense", "ff": 16, "limit": 1.0},
              "mixer": dict(heads=6, kv_heads=3, dim=10, vdim=14, scale=0.25, kv_from=1)}
    return dict(architecture="Norelix", vocab=50, width=24, norm={"eps": 1e-5},
                layers=[par, att, copy.deepcopy(par), shared])


def test_config_round_trip_and_registry(tmp_path):
    cfg = NorelixConfig.from_dict(raw_config())
    assert cfg.norm_eps == 1e-5 and len(cfg.layers) == 4 and cfg.kv_source(3) == 1 and cfg.kv_source(1) == 1
    write_random_model(str(tmp_path), cfg, seed=0, std=0.1)
    again = load_config(str(tmp_path))
    assert isinstance(again, NorelixConfig) and again == NorelixConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("vdim"), "left.vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "right.conv"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "mlp.limit"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "q_temp.every"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),          # not an attention layer
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),          # itself
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "kv_from"),            # other sizes than its source
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError) as e:
        NorelixConfig.from_dict(raw)
    assert word in str(e.value)


def test_optional_groups_switch_their_mechanism_off():
    raw = raw_config()
    raw["layers"][0]["mixer"]["left"].pop("mask")
    raw["layers"][0]["mixer"]["left"].pop("rot")
    raw["layers"][1]["mixer"].pop("q_temp")
    mdef = build_model_def(NorelixConfig.from_dict(raw))
    left = mdef.blocks[0].mixer.left
    assert left.window is None and left.keep_first == 0 and left.qk_position is None
    assert mdef.blocks[1].mixer.q_temp is None and mdef.blocks[2].mixer.left.window == 20


def test_tensor_names_shapes_and_cache_needs():
    mdef = build_model_def(NorelixConfig.from_dict(raw_config()))
    specs = {s.name: tuple(s.shape) for s in mdef.param_specs()}
    assert specs["embed"] == (50, 24) and specs["head"] == (50, 24) and specs["final.norm"] == (24,)
    assert specs["l0.mix.left.q"] == (32, 24) and specs["l0.mix.left.k.b"] == (16,) and specs["l0.mix.left.v"] == (24, 24)
    assert specs["l0.mix.left.o"] == (24, 48) and "l0.mix.left.o.b" not in specs
    assert specs["l0.mix.right.q"] == (12, 24) and specs["l0.mix.right.v.conv"] == (40, 3) and specs["l0.mix.right.b"] == (4, 24)
    assert specs["l0.mix.right.A_log"] == (4,) and specs["l0.mix.right.dt_bias"] == (24,) and specs["l0.mix.right.norm"] == (10,)
    # the low-rank pairs' inner size is the checkpoint's own
    assert specs["l0.mix.right.a1"][0] < 0 and specs["l0.mix.right.a2"] == (24, specs["l0.mix.right.a1"][0])
    assert specs["l1.mix.g"] == (84, 24) and specs["l1.mix.o.b"] == (24,) and "l1.norm2" not in specs and "l1.mlp.gate" not in specs
    assert "l3.mix.k" not in specs and "l3.mix.v.b" not in specs and specs["l3.mix.q.b"] == (60,)
    assert specs["l3.mlp.gate.b"] == (16,) and specs["l3.mlp.down.b"] == (24,)
    # three cache entries for four layers: the last layer reads the second one's pages
    needs = mdef.cache_specs()
    assert len(needs) == 3
    pages, (tails, mats) = needs[0]
    assert pages == PagedKVSpec(2, 8, 20, value_dim=12, keep_first=6)
    assert tails == StateSpec((2, 12 + 12 + 40)) and mats == StateSpec((4, 6, 10))
    assert needs[1] == PagedKVSpec(3, 10, None, value_dim=14)
    order = mdef.layer_order
    assert [(o.block, o.cache, o.writes_cache) for o in order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]


def test_cache_entries_views_and_zeroed_slots():
    mdef = build_model_def(NorelixConfig.from_dict(raw_config()))
    m = CacheManager(mdef.cache_specs(), torch.float32, "cpu", page_size=4, num_pages=16, max_seqs=2, max_seq_len=64)
    pages, (tails, mats) = m.entries()[0].view()
    assert isinstance(pages, PagedCacheView) and isinstance(tails, StateView) and isinstance(mats, StateView)
    assert tails.state.shape == (2, 2, 64) and mats.state.shape == (2, 4, 6, 10) and mats.state.dtype == torch.float32
    s = m.alloc_slot()
    mats.state[s].fill_(1.0)
    tails.state[s].fill_(1.0)
    m.free_slot(s)
    assert m.alloc_slot() == s and float(mats.state[s].abs().sum()) == 0.0 and float(tails.state[s].abs().sum()) == 0.0


@pytest.mark.parametrize("window,keep,ps", [(20, 6, 4), (9, 1, 8), (16, 0, 4), (5, 17, 4)])
def test_window_releases_pages_behind_it_but_not_the_kept_first(window, keep, ps):
    m = CacheManager([PagedKVSpec(1, 8, window, value_dim=4, keep_first=keep)], torch.float32, "cpu", page_size=ps,
                     num_pages=24, max_seqs=1, max_seq_len=400)
    s = m.alloc_slot()
    g = m.groups[0]
    kept_pages = (keep + ps - 1) // ps
    sizes = (7, 2, 1, 1, 30, 3)
    start, k, held = 0, 0, []
    while start < 300:
        n = sizes[k % len(sizes)]
        k += 1
        assert m.reserve(s, start, start + n)
        have = set(g.pages[s])
        # every key that a query of this portion sees has its page
        for p in range(start, start + n):
            for j in range(p + 1):
                if p - j < window or j < keep:
                    assert j // ps in have, (p, j)
        m.commit(s, start + n)
        start += n
        held.append(g.pool.num_held)
        assert all(j in g.pages[s] for j in range(min(kept_pages, (start + ps - 1) // ps)))
    assert max(held) <= kept_pages + (window + 30 + ps - 1) // ps + 2
    m.check()
    m.free_slot(s)
    assert g.pool.num_held == 0


# ------------------------------------------------------------------------------------------ the oracle's own mechanisms
def test_plain_mask_rotation_temperature_and_sink():
    seen = pn.seen_window(12, 4, 2)
    assert seen[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert seen[3].tolist() == [True] * 4 + [False] * 8 and not seen[5, 6]
    # rotating by position p and taking the dot product depends on the distance only
    rng = np.random.default_rng(0)
    u, v = rng.normal(size=(1, 1, 6)), rng.normal(size=(1, 1, 6))
    a = (pn.rotate_halves(u, [7], 4, 10.0) * pn.rotate_halves(v, [3], 4, 10.0)).sum()
    b = (pn.rotate_halves(u, [14], 4, 10.0) * pn.rotate_halves(v, [10], 4, 10.0)).sum()
    assert abs(a - b) < 1e-12 and np.allclose(pn.rotate_halves(u, [9], 4, 10.0)[..., 4:], u[..., 4:])
    assert np.allclose(pn.temperature([0, 3, 4, 9], 0.5, 5), [1.0, 1.0, 1 + 0.5 * np.log(2.0), 1 + 0.5 * np.log(3.0)])
    w = pn.softmax_rows(np.zeros((1, 3)), np.array([[True, True, False]]), one_more=True)
    assert np.allclose(w, [[1 / 3, 1 / 3, 0.0]])


def test_plain_delta_rule_overwrites_a_key_and_decays():
    """Writing along a unit key with strength 1 stores the value exactly; a second write along the same key replaces
    it; a decay of one half per token halves what a later query reads."""
    d, vd = 4, 3
    k = np.zeros((3, d)); k[:, 1] = 1.0
    v = np.array([[1.0, 2.0, 3.0], [5.0, 5.0, 5.0], [0.0, 0.0, 0.0]])
    q = k.copy()
    o = pn.delta_rule(q, k, v, np.ones((3, d)), np.array([1.0, 1.0, 0.0]))
    assert np.allclose(o, [[1, 2, 3], [5, 5, 5], [5, 5, 5]])
    o = pn.delta_rule(q, k, v, np.full((3, d), 0.5), np.array([1.0, 0.0, 0.0]))
    assert np.allclose(o, [[1, 2, 3], [0.5, 1, 1.5], [0.25, 0.5, 0.75]])
    f = np.array([[0.0, 1.0], [2.0, 3.0]])
    u = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]])
    assert np.allclose(pn.causal_conv(u, f), [[1, 30], [2, 80], [3, 130]])
