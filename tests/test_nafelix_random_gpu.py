"""Randomly drawn Nafelix configurations through the trace replay against the plain implementation: sizes that are and
are not multiples of the kernels' tiles, one head to many, one to six streams, with and without convolutions, loop,
mask, rotation and feed-forward, layers in any order, in both types, as a mixed batch with pages and slots used again
and in portions down to two tokens."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import helpers
import plain_nafelix as pn

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    width = int(pick(24, 40, 64, 72, 96, 100))

    def attention():
        kv = int(pick(1, 1, 2, 3, 4))
        dim = int(pick(4, 8, 16, 24, 10, 32, 64))
        mx = dict(heads=kv * int(pick(1, 1, 2, 4, 8)), kv_heads=kv, dim=dim, vdim=int(pick(4, 8, 16, 20, 48)),
                  scale=float(pick(0.2, 0.35, 0.5, dim ** -0.5)))
        if rng.random() < 0.85:
            mx["mask"] = {"size": int(pick(1, 2, 7, 16, 17, 31, 33, 64, 100, 500))}
        if rng.random() < 0.85:
            mx["rot"] = {"dims": int(rng.integers(0, dim // 2 + 1)) * 2, "base": float(pick(10.0, 100.0, 10000.0, 3e5))}
        return mx

    def mlp():
        kind = pick("dense", "moe", "moe", None)
        if kind == "dense":
            return {"kind": "dense", "ff": int(pick(16, 40, 64, 100))}
        if kind == "moe":
            n = int(pick(1, 2, 4, 7, 16))
            return {"kind": "moe", "expert": {"ff": int(pick(8, 16, 24, 20)), "limit": float(pick(0.5, 1.5, 7.0))},
                    "router": {"experts": n, "top": int(rng.integers(1, min(n, 4) + 1))}}
        return None

    n_layers = int(rng.integers(1, 5))
    layers = []
    for _ in range(n_layers):
        if rng.random() < 0.55:
            qk = int(pick(1, 2, 3))
            right = dict(heads=qk * int(pick(1, 2, 3)), kv_heads=qk, dim=int(pick(4, 8, 16, 24, 40)),
                         vdim=int(pick(4, 8, 16, 20)), conv=int(pick(1, 2, 3, 4, 6)))
            layers.append({"type": "parallel", "mixer": {"left": attention(), "right": right}, "mlp": mlp()})
        else:
            layers.append({"type": "attention", "mixer": attention(), "mlp": mlp()})
    cfg = dict(architecture="Nafelix", vocab=int(pick(64, 130, 257)), width=width, streams=int(pick(1, 2, 3, 4, 6)),
               norm={"eps": float(pick(1e-5, 1e-4, 3e-6))}, layers=layers)
    if rng.random() < 0.8:
        cfg["canon"] = {"taps": int(pick(1, 2, 3, 5))}
    if rng.random() < 0.7:
        start = int(rng.integers(0, n_layers))
        stop = int(rng.integers(start + 1, n_layers + 1))
        cfg["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return cfg, float(pick(0.08, 0.1, 0.12)), int(pick(4, 8, 16, 16))


def write_model(path, cfg_dict, seed, std):
    from swifttransformer_b200.config import NafelixConfig, save_config
    from swifttransformer_b200.models import build_model_def
    from swifttransformer_b200.weights.random_init import random_tensors
    from swifttransformer_b200.weights.safetensors_io import write_safetensors
    cfg = NafelixConfig.from_dict(cfg_dict)
    save_config(cfg, path)
    n, tensors = cfg.streams, []
    for s, t in random_tensors(build_model_def(cfg).param_specs(), seed, std, "cpu"):
        f = t.float()
        if s.name.endswith(".A_log"):
            f = f - 3.0
        elif s.name.endswith(".router"):
            f = f * 6                                    # loud routers: the choice does not hang on the last bit
        elif s.name.endswith((".sink", ".act")):
            f = f / std * 1.5
        elif s.name.endswith(".b") and t.dim() == 1:
            f = f * 3
        elif s.name.endswith(".talk"):
            f = torch.eye(t.shape[0]) + f / std * 0.3
        elif s.name.endswith((".hc1.in", ".hc2.in")):
            f = 1.0 / n + f / std * 0.1
        elif s.name.endswith((".hc1.out", ".hc2.out")):
            f = 1.0 + f / std * 0.15
        elif s.name.endswith((".hc1.mix", ".hc2.mix")):
            f = torch.eye(n) + f / std * 0.1
        elif s.name.endswith((".canon1", ".canon2")):
            f = f / std * 0.3
        tensors.append((s.name, f.to(torch.bfloat16)))
    write_safetensors(os.path.join(path, "model.safetensors"), tensors)
    return path


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(200, 216)))
def test_random_configuration_as_a_mixed_batch_and_in_portions(tmp_path, seed, dtype):
    from swifttransformer_b200.engine.replay import TraceSession
    cfg, std, page_size = draw(seed)
    path = write_model(str(tmp_path / "m"), cfg, seed, std)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab"], n, seed=seed + i) for i, n in enumerate((150, 1, 37, 64, 19))}
    pcfg, w = pn.load_model(path)
    refs = {rid: pn.forward(pcfg, w, toks) for rid, toks in reqs.items()}
    for steps in (helpers.trace_mixed(reqs, seed=seed, max_live=3), helpers.trace_portions(reqs)):
        s = TraceSession(path, dtype, helpers.live_token_need(steps), page_size=page_size, max_requests=3)
        got = helpers.replay(s, steps)
        errs = []
        for rid in reqs:
            scale = np.abs(refs[rid]).max()
            err = np.abs(got[rid] - refs[rid]).max(axis=1) / scale
            if dtype == "float32":
                assert err.max() < 4e-5, (seed, cfg, rid, int(np.argmax(err)), float(err.max()))
            errs.append(err)
        err = np.concatenate(errs)
        if dtype == "bfloat16":
            # Where two router scores lie within the activations' rounding a token goes to another expert, and what
            # it then writes into the recurrence's state stays with every later token of its request: the bound is on
            # the typical position, and nothing may be wild.  (float32 above is held at every position.)
            assert np.isfinite(err).all() and np.median(err) < 3e-2 and err.max() < 1.0, \
                (seed, cfg, float(np.median(err)), float((err > 6e-2).mean()), float(err.max()))
        s.cache.check()
        assert all(g.pool.num_held == 0 for g in s.cache.groups)
