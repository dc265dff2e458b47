"""The Nafelix design's host side on the CPU: configuration, tensor names, the order of layer runs with a looped
stretch, the cache entries of a block that keeps convolution states beside its mixer's pages and states, and the plain
implementation's own mechanisms against closed forms.  (What runs kernels is in test_nafelix_gpu.py.)"""
from __future__ import annotations

import copy
import json

import numpy as np
import pytest
import torch

import plain_nafelix as pn
from swifttransformer_b200.cache.manager import CacheManager, PagedCacheView, StateView
from swifttransformer_b200.config import ConfigError, NafelixConfig, load_config
from swifttransformer_b200.models import build_model_def, write_random_model
from swifttransformer_b200.parts.base import PagedKVSpec, StateSpec


def raw_config():
    left = dict(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.3, mask={"size": 20}, rot={"dims": 4, "base": 100.0})
    right = dict(heads=4, kv_heads=2, dim=6, vdim=10, conv=3)
    par = {"type": "parallel", "mlp": {"kind": "dense", "ff": 40}, "mixer": {"left": left, "right": right}}
    att = {"type": "attention", "mlp": None,
           "mixer": dict(heads=6, kv_heads=3, dim=10, vdim=14, scale=0.2, mask={"size": 7}, rot={"dims": 10, "base": 9.0})}
    routed = copy.deepcopy(par)
    routed["mlp"] = {"kind": "moe", "expert": {"ff": 16, "limit": 1.5}, "router": {"experts": 5, "top": 2}}
    return dict(architecture="Nafelix", vocab=50, width=24, streams=3, norm={"eps": 1e-5}, canon={"taps": 4},
                loop={"start": 1, "stop": 3, "times": 2}, layers=[par, att, routed, copy.deepcopy(att)])


def test_config_round_trip_and_registry(tmp_path):
    cfg = NafelixConfig.from_dict(raw_config())
    assert cfg.norm_eps == 1e-5 and cfg.streams == 3 and cfg.canon_taps == 4 and cfg.loop == (1, 3, 2)
    assert cfg.layer_runs() == [0, 1, 2, 1, 2, 3]
    write_random_model(str(tmp_path), cfg, seed=0, std=0.1)
    again = load_config(str(tmp_path))
    assert isinstance(again, NafelixConfig) and again == NafelixConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["canon"].update(taps=9), "canon.taps"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].pop("times"), "loop.times"),
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("vdim"), "left.vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "right.conv"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "mixer.scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["layers"][2]["mlp"]["expert"].pop("limit"), "expert.limit"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=6), "router.top"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError) as e:
        NafelixConfig.from_dict(raw)
    assert word in str(e.value)


def test_optional_groups_switch_their_mechanism_off():
    raw = raw_config()
    raw["layers"][0]["mixer"]["left"].pop("mask")
    raw["layers"][0]["mixer"]["left"].pop("rot")
    for key in ("canon", "loop", "streams"):
        raw.pop(key)
    cfg = NafelixConfig.from_dict(raw)
    mdef = build_model_def(cfg)
    left = mdef.blocks[0].mixer.left
    assert left.window is None and left.qk_position is None and mdef.blocks[2].mixer.left.window == 20
    assert cfg.streams == 1 and cfg.layer_runs() == [0, 1, 2, 3]
    names = {s.name for s in mdef.param_specs()}
    assert "l0.canon1" not in names and "l0.hc1.mix" in names
    # no convolution: the block keeps no state of its own
    tail1, _, tail2 = mdef.cache_specs()[0]
    assert tail1 is None and tail2 is None


def test_tensor_names_shapes_and_cache_needs():
    mdef = build_model_def(NafelixConfig.from_dict(raw_config()))
    specs = {s.name: tuple(s.shape) for s in mdef.param_specs()}
    assert specs["embed"] == (50, 24) and specs["head"] == (50, 24) and specs["final.norm"] == (24,)
    assert specs["l0.mix.left.q"] == (32, 24) and specs["l0.mix.left.v"] == (24, 24) and "l0.mix.left.q.b" not in specs
    assert specs["l0.mix.left.talk"] == (4, 4) and specs["l0.mix.left.sink"] == (4,) and specs["l0.mix.left.g"] == (4, 24)
    assert specs["l0.mix.left.o"] == (24, 48) and specs["l0.mix.left.out"] == (24,) and specs["l0.mix.right.out"] == (24,)
    assert specs["l0.mix.right.q"] == (12, 24) and specs["l0.mix.right.v.conv"] == (40, 3) and specs["l0.mix.right.b"] == (4, 24)
    assert specs["l0.mix.right.a"] == (4, 24) and specs["l0.mix.right.dt_bias"] == (4,) and specs["l0.mix.right.g"] == (40, 24)
    assert specs["l0.mix.right.A_log"] == (4,) and specs["l0.mix.right.norm"] == (10,)
    assert specs["l0.mlp.up"] == (40, 24) and specs["l0.mlp.down"] == (24, 40) and specs["l0.mlp.act"] == (2,)
    assert specs["l0.hc1.in"] == (3,) and specs["l0.hc2.mix"] == (3, 3) and specs["l0.canon2"] == (24, 4)
    assert specs["l1.mix.q.b"] == (60,) and specs["l1.mix.g"] == (84, 24) and specs["l1.mix.sink"] == (6,)
    assert "l1.norm2" not in specs and "l1.hc2.in" not in specs and "l1.canon2" not in specs and "l1.mix.talk" not in specs
    assert specs["l2.mlp.router"] == (5, 24) and specs["l2.mlp.e4.gate"] == (16, 24) and specs["l2.mlp.e0.down"] == (24, 16)
    # six layer runs, six cache entries: every run of a looped layer has its own
    needs = mdef.cache_specs()
    assert [(o.block, o.cache) for o in mdef.layer_order] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (3, 5)]
    tail1, (pages, (conv, mats)), tail2 = needs[0]
    assert tail1 == tail2 == StateSpec((3, 24)) and pages == PagedKVSpec(2, 8, 20, value_dim=12)
    assert conv == StateSpec((2, 12 + 12 + 40)) and mats == StateSpec((4, 6, 10))
    assert needs[1] == (StateSpec((3, 24)), PagedKVSpec(3, 10, 7, value_dim=14), None) and needs[1] == needs[3]


def test_cache_entries_views_and_zeroed_slots():
    mdef = build_model_def(NafelixConfig.from_dict(raw_config()))
    m = CacheManager(mdef.cache_specs(), torch.float32, "cpu", page_size=4, num_pages=16, max_seqs=2, max_seq_len=64)
    tail1, (pages, (conv, mats)), tail2 = m.entries()[2].view()
    assert isinstance(pages, PagedCacheView) and all(isinstance(v, StateView) for v in (tail1, tail2, conv, mats))
    assert tail1.state.shape == (2, 3, 24) and tail1.state is not tail2.state and mats.state.shape == (2, 4, 6, 10)
    # the two runs of a looped layer do not share anything
    again = m.entries()[4].view()
    assert again[0].state is not tail1.state and again[1][1][1].state is not mats.state
    assert again[1][0].block_table is pages.block_table and again[1][0].layer != pages.layer
    s = m.alloc_slot()
    for v in (tail1, tail2, conv, mats):
        v.state[s].fill_(1.0)
    m.free_slot(s)
    assert m.alloc_slot() == s and all(float(v.state[s].abs().sum()) == 0.0 for v in (tail1, tail2, conv, mats))
    assert m.entries()[1].view()[2] is None


# ------------------------------------------------------------------------------------------ the oracle's own mechanisms
def test_plain_window_rotation_and_extra_term():
    seen = pn.seen_window(12, 4)
    assert seen[11].tolist() == [False] * 8 + [True] * 4 and seen[2].tolist() == [True] * 3 + [False] * 9
    assert pn.seen_window(5, None)[4].all() and not pn.seen_window(5, None)[2, 3]
    rng = np.random.default_rng(0)
    u, v = rng.normal(size=(1, 1, 6)), rng.normal(size=(1, 1, 6))
    a = (pn.rotate_halves(u, [7], 4, 10.0) * pn.rotate_halves(v, [3], 4, 10.0)).sum()
    b = (pn.rotate_halves(u, [14], 4, 10.0) * pn.rotate_halves(v, [10], 4, 10.0)).sum()
    assert abs(a - b) < 1e-12 and np.allclose(pn.rotate_halves(u, [9], 4, 10.0)[..., 4:], u[..., 4:])
    # dimension 0 is paired with dimension 2 when four dimensions turn
    e0 = np.zeros((1, 1, 6)); e0[..., 0] = 1.0
    r = pn.rotate_halves(e0, [1], 4, 10.0)[0, 0]
    assert np.allclose(r[[0, 2]], [np.cos(1.0), np.sin(1.0)]) and np.allclose(r[[1, 3, 4, 5]], 0.0)
    w = pn.softmax_with_sink(np.zeros((2, 1, 3)), np.array([[True, True, False]]), np.log(np.array([1.0, 2.0])))
    assert np.allclose(w[0], [[1 / 3, 1 / 3, 0.0]]) and np.allclose(w[1], [[1 / 4, 1 / 4, 0.0]])


def test_plain_mixing_of_heads_keeps_each_head_on_its_own_values():
    """Head 0 given head 1's weights reads the values of its own group under head 1's softmax."""
    T = np.array([[0.0, 1.0], [1.0, 0.0]])
    P = np.zeros((2, 1, 2)); P[0, 0] = [1.0, 0.0]; P[1, 0] = [0.25, 0.75]
    v = np.zeros((2, 2, 1)); v[:, 0, 0] = [10.0, 20.0]; v[:, 1, 0] = [1.0, 2.0]
    o = pn.apply_weights(np.einsum("ab,bij->aij", T, P), v)
    assert np.allclose(o[0, :, 0], [0.25 * 10 + 0.75 * 20, 1.0])


def test_plain_delta_rule_overwrites_a_key_and_decays():
    d = 4
    k = np.zeros((3, 1, d)); k[:, 0, 1] = 1.0
    v = np.array([[1.0, 2.0, 3.0], [5.0, 5.0, 5.0], [0.0, 0.0, 0.0]])[:, None, :]
    ones = np.ones((3, 1))
    o = pn.delta_rule(k, k, v, ones, np.array([[1.0], [1.0], [0.0]]))
    assert np.allclose(o[:, 0], [[1, 2, 3], [5, 5, 5], [5, 5, 5]])
    o = pn.delta_rule(k, k, v, 0.5 * ones, np.array([[1.0], [0.0], [0.0]]))
    assert np.allclose(o[:, 0], [[1, 2, 3], [0.5, 1, 1.5], [0.25, 0.5, 0.75]])
    f = np.array([[0.0, 1.0], [2.0, 3.0]])
    u = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]])
    assert np.allclose(pn.causal_conv(u, f), [[1, 30], [2, 80], [3, 130]])


def test_plain_streams_activation_router_and_loop():
    xs = np.arange(12.0).reshape(2, 3, 2)
    w = {"hc.in": np.array([1.0, 0.0]), "hc.out": np.array([0.0, 2.0]), "hc.mix": np.array([[0.0, 1.0], [1.0, 0.0]])}
    y = np.ones((3, 2))
    new = pn.streams_update(xs, y, w, "hc")
    assert np.allclose(new[0], xs[1]) and np.allclose(new[1], xs[0] + 2.0)        # mix is indexed [from, to]
    assert np.isclose(pn.xielu(np.array(2.0), 0.0, 0.0), np.log(2.0) * 4 + 1.0)
    assert np.isclose(pn.xielu(np.array(-1.0), 0.0, 0.0), (0.5 + np.log(2.0)) * (np.exp(-1.0) - 1 + 1) - 0.5)
    chosen, weights = pn.route(np.array([[1.0, 0.0]]), np.array([[0.0, 0.0], [np.log(3.0), 0.0], [np.log(6.0), 0.0]]), 2)
    assert chosen.tolist() == [[2, 1]] and np.allclose(weights, [[2 / 3, 1 / 3]])
    assert np.allclose(pn.clamped_unit(np.array([5.0]), np.array([-7.0]), 2.0), 2.0 * pn.sigmoid(3.404) * (-1.0))
    assert pn.layer_runs({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert pn.layer_runs({"layers": [0] * 2}) == [0, 1]
