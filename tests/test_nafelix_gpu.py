"""The Nafelix design on the GPU against the plain implementation (tests/plain_nafelix.py).

Mechanisms alone (the kernels driven directly, with inputs made so that a single key, an edge, a stream or the
extra term decides the result), then whole models of several small configurations through the trace replay (whole
prompts, token-by-token decoding, portions down to two tokens, mixed batches with pages and slots used again) and
through ``LLMEngine.generate`` and the programs.
"""
from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_nafelix as pn

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def bf16_round(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(torch.bfloat16).double().numpy()


class Step:
    """The index arrays of one step for (slot, start, n) entries, with padding tokens at position -1 and padding
    requests behind, as the step function lays them out."""

    def __init__(self, entries, pad_tokens=0, pad_requests=0):
        pos, seq, q_start, slots, starts = [], [], [0], [], []
        for i, (slot, start, n) in enumerate(entries):
            pos += list(range(start, start + n))
            seq += [i] * n
            q_start.append(q_start[-1] + n)
            slots.append(slot)
            starts.append(start)
        self.n = len(pos)
        pos += [-1] * pad_tokens
        seq += [0] * pad_tokens
        q_start += [self.n] * pad_requests
        slots += [0] * pad_requests
        starts += [0] * pad_requests
        self.n_rows, self.n_seqs = len(pos), len(entries) + pad_requests
        self.positions, self.seq, self.q_start, self.slots = ints(pos), ints(seq), ints(q_start), ints(slots)
        self.start_pos = ints(starts)


def portions(total, sizes):
    out, pos, k = [], 0, 0
    while pos < total:
        n = min(sizes[k % len(sizes)], total - pos)
        out.append((pos, n))
        pos += n
        k += 1
    return out


# ------------------------------------------------------------------------------------------ residual streams
@pytest.mark.parametrize("n,width", [(1, 20), (3, 48), (4, 64), (8, 33)])
def test_streams_read_and_write(n, width):
    """The mixture a sub-layer reads with its norm, the update of all copies at once from the old ones, the copies'
    start and their sum, against the plain functions; rows of padding tokens are not read."""
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(n * width)
    T = 9
    xs = rng.normal(size=(n, T, width))
    w = {"hc.in": rng.normal(size=n), "hc.mix": rng.normal(size=(n, n)), "hc.out": rng.normal(size=n),
         "norm": 1 + 0.1 * rng.normal(size=width), "canon": np.zeros((width, 1))}
    lanes = dev(xs)
    pos = list(range(T - 1)) + [-1]
    h = ops.hc_read_norm(lanes, dev(w["hc.in"]), dev(w["norm"]), 1e-3, ints(pos)).cpu().numpy()
    ref = pn.sublayer_input(xs, w, "hc", "norm", "canon", 1e-3)
    assert np.abs(h[:T - 1] - ref[:T - 1]).max() < 1e-5 * np.abs(ref).max()
    for ydt in (torch.float32, torch.bfloat16):
        y = bf16_round(rng.normal(size=(T, width)))
        lanes = dev(xs)
        ops.hc_write(lanes, dev(w["hc.mix"]), dev(w["hc.out"]), dev(y, ydt))
        ref = pn.streams_update(xs, y, w, "hc")
        assert np.abs(lanes.cpu().numpy() - ref).max() < 1e-5 * np.abs(ref).max()
    # the update and the next sub-layer's read in one pass: the same copies and the same normed mixture; the padding
    # token's row is left alone
    w2 = {"hc.in": rng.normal(size=n), "norm": 1 + 0.1 * rng.normal(size=width)}
    for ydt in (torch.float32, torch.bfloat16):
        y = bf16_round(rng.normal(size=(T, width)))
        lanes = dev(xs)
        h = ops.hc_write_read_norm(lanes, dev(w["hc.mix"]), dev(w["hc.out"]), dev(y, ydt), dev(w2["hc.in"]), dev(w2["norm"]),
                                   1e-3, ints(pos)).cpu().numpy()
        new = pn.streams_update(xs, y, w, "hc")
        got = lanes.cpu().numpy()
        assert np.abs(got[:, :T - 1] - new[:, :T - 1]).max() < 1e-5 * np.abs(new).max() and np.array_equal(got[:, T - 1], xs[:, T - 1].astype(np.float32))
        ref = pn.sublayer_input(new, w2, "hc", "norm", "none", 1e-3)
        assert np.abs(h[:T - 1] - ref[:T - 1]).max() < 2e-5 * np.abs(ref).max()
    # a mixing matrix that swaps two copies shows an update that reads a copy it has already written
    if n >= 2:
        swap = np.ascontiguousarray(np.eye(n)[:, [1, 0] + list(range(2, n))])
        lanes = dev(xs)
        ops.hc_write(lanes, dev(swap), dev(np.zeros(n)), dev(np.zeros((T, width))))
        got = lanes.cpu().numpy()
        assert np.abs(got[0] - xs[1]).max() < 1e-6 and np.abs(got[1] - xs[0]).max() < 1e-6
    x = dev(xs[0])
    spread = ops.hc_spread(x, n)
    assert torch.equal(spread, x.unsqueeze(0).expand(n, T, width))
    assert np.abs(ops.hc_sum(dev(xs)).cpu().numpy() - xs.sum(0)).max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,width,taps", [(3, 44, 2), (4, 64, 5), (1, 20, 3)])
def test_single_token_steps_update_read_norm_and_convolve_in_one_kernel(dtype, n, width, taps):
    """Three requests decoded side by side for several steps through ``hc_step_conv`` (with and without a pending
    update), a padding token beside them: the sub-layer's input equals norm + convolution of the plain functions over
    each request's whole history, and the states of other slots are left alone."""
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(n * width + taps)
    B, steps, slots = 3, 7, [2, 0, 3]
    w = {"hc.in": rng.normal(size=n), "hc.mix": np.eye(n) + 0.2 * rng.normal(size=(n, n)), "hc.out": 1 + 0.2 * rng.normal(size=n),
         "norm": 1 + 0.1 * rng.normal(size=width), "canon": rng.normal(size=(width, taps)) * 0.5}
    state = torch.zeros((5, taps - 1, width), device="cuda")
    state[1] = 7.0
    xs = rng.normal(size=(steps, n, B, width))            # the copies' rows each step brings (before the update)
    ys = bf16_round(rng.normal(size=(steps, B, width)))
    hist = [[] for _ in range(B)]
    for k in range(steps):
        lanes = dev(np.concatenate([xs[k], np.full((n, 1, width), 3.0)], axis=1))
        st = Step([(slots[b], k, 1) for b in range(B)], pad_tokens=1)
        pending = None if k % 3 == 0 else (dev(w["hc.mix"]), dev(w["hc.out"]), dev(np.concatenate([ys[k], np.zeros((1, width))]), TD[dtype]))
        out = torch.full((B + 1, width), 5.0, dtype=TD[dtype], device="cuda")
        ops.hc_step_conv(lanes, pending, dev(w["hc.in"]), dev(w["norm"]), 1e-4, dev(w["canon"]), state, out, st.positions,
                         st.seq, st.slots)
        new = pn.streams_update(xs[k], ys[k], w, "hc") if pending is not None else xs[k]
        assert np.abs(lanes.cpu().numpy()[:, :B] - new).max() < 1e-5 * np.abs(new).max()
        assert np.all(lanes.cpu().numpy()[:, B] == 3.0) and np.all(out.float().cpu().numpy()[B] == 5.0)
        got = out.float().cpu().numpy()
        for b in range(B):
            u = np.einsum("s,sw->w", w["hc.in"], new[:, b])
            hist[b].append(pn.rms_unit(u, 1e-4) * w["norm"])
            h = np.stack(hist[b])
            ref = (h + pn.causal_conv(h, w["canon"]))[-1]
            tol = 2e-5 if dtype == "float32" else 1e-2
            assert np.abs(got[b] - ref).max() < tol * np.abs(ref).max(), (k, b)
    assert torch.all(state[1] == 7.0) and float(state[4].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_of_normed_results_and_two_sided_activation(dtype):
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(4)
    for width in (20, 48, 257):
        a, b = bf16_round(rng.normal(size=(7, width)) * 3), rng.normal(size=(7, width)) * 0.01
        wa, wb = 1 + 0.2 * rng.normal(size=width), 1 + 0.2 * rng.normal(size=width)
        got = ops.norm_pair_sum(dev(a, TD[dtype]), dev(wa), 0.5, dev(b), dev(wb), 0.5, 1e-4).cpu().numpy()
        ref = 0.5 * (pn.rms_unit(a, 1e-4) * wa + pn.rms_unit(b.astype(np.float32).astype(np.float64), 1e-4) * wb)
        assert np.abs(got - ref).max() < 2e-5 * np.abs(ref).max()
    z = bf16_round(np.concatenate([rng.normal(size=500) * 3, [0.0, -0.0, 30.0, -30.0]]))
    for p, q in ((0.3, -0.7), (-2.0, 1.5), (0.0, 0.0)):
        got = ops.xielu(dev(z, TD[dtype]), float(pn.softplus(p)), float(0.5 + pn.softplus(q))).float().cpu().numpy()
        ref = pn.xielu(z, p, q)
        tol = 1e-5 if dtype == "float32" else 1e-2
        assert np.abs(got - ref).max() < tol * np.abs(ref).max()


# ------------------------------------------------------------------------------------------ attention with mixed heads
class TalkCase:
    """Queries, keys, values, gate logits, sinks and a mixing matrix; keys and values stand in a paged pool whose
    pages are dealt out of order and whose unused rows hold large numbers."""

    def __init__(self, lengths, H, G, d, vd, ps, seed, dtype, window, talk=True, sinks=True, gate="head"):
        rng = np.random.default_rng(seed)
        self.H, self.G, self.d, self.vd, self.ps, self.dtype, self.window = H, G, d, vd, ps, dtype, window
        self.lengths = list(lengths)
        self.q = [bf16_round(rng.normal(size=(n, H, d))) for n in lengths]
        self.k = [bf16_round(rng.normal(size=(n, G, d))) for n in lengths]
        self.v = [bf16_round(rng.normal(size=(n, G, vd))) for n in lengths]
        self.gate_kind = gate
        gw = H if gate == "head" else H * vd
        self.gate = [bf16_round(rng.normal(size=(n, gw))) for n in lengths] if gate else None
        self.talk = (np.eye(H) + 0.5 * rng.normal(size=(H, H))).astype(np.float32).astype(np.float64) if talk else None
        self.sinks = rng.normal(size=H).astype(np.float32).astype(np.float64) if sinks else None
        self.scale = 0.9 / np.sqrt(d)
        per = [(n + ps - 1) // ps for n in lengths]
        self.max_pages = max(per) + 1
        self.n_pages = sum(per) + 3
        order = rng.permutation(self.n_pages)
        self.table = np.full((len(lengths) + 1, self.max_pages), -1, dtype=np.int32)
        self.slot = [len(lengths) - i for i in range(len(lengths))]
        at = 0
        for i, c in enumerate(per):
            self.table[self.slot[i], :c] = order[at:at + c]
            at += c

    def write_pool(self):
        G, ps, d, vd = self.G, self.ps, self.d, self.vd
        keys = np.full((self.n_pages, G, ps, d), 3e4)
        vals = np.full((self.n_pages, G, ps, vd), 3e4)
        for i, n in enumerate(self.lengths):
            for p in range(n):
                page = self.table[self.slot[i], p // ps]
                keys[page, :, p % ps] = self.k[i][p]
                vals[page, :, p % ps] = self.v[i][p]
        flat = np.concatenate([keys.reshape(self.n_pages, -1), vals.reshape(self.n_pages, -1)], axis=1)
        pool = np.full((self.n_pages, 2, flat.shape[1]), 3e4)
        pool[:, 1] = flat
        self.pool = dev(pool, TD[self.dtype])

    def reference(self, i):
        n = self.lengths[i]
        seen = pn.seen_window(n, self.window or None)
        sinks = self.sinks if self.sinks is not None else np.full(self.H, -np.inf)
        P = pn.attention_weights(self.q[i], self.k[i], seen, self.scale, sinks)
        if self.talk is not None:
            P = np.einsum("ab,bij->aij", self.talk, P)
        o = pn.apply_weights(P, self.v[i])
        if self.gate is not None:
            g = pn.sigmoid(self.gate[i])
            o = o * (g[:, :, None] if self.gate_kind == "head" else g.reshape(n, self.H, self.vd))
        return o.reshape(n, -1)

    def drop_pages_out_of_sight(self, i, pos):
        table = self.table.copy()
        if self.window:
            for page in range(max(0, pos - self.window + 1) // self.ps):
                table[self.slot[i], page] = -1
        return table

    def run(self, entries, kernel, pad_tokens=0, table=None):
        from swifttransformer_b200 import ops
        H, G, d, vd = self.H, self.G, self.d, self.vd
        st = Step([(self.slot[i], s, n) for i, s, n in entries], pad_tokens=pad_tokens)
        q = np.concatenate([self.q[i][s:s + n] for i, s, n in entries] + [np.full((pad_tokens, H, d), 50.0)])
        qd = dev(q.reshape(st.n_rows, -1), TD[self.dtype])
        wide, gate_off = None, 0
        if self.gate is not None:
            g = np.concatenate([self.gate[i][s:s + n] for i, s, n in entries] + [np.zeros((pad_tokens, self.gate[0].shape[1]))])
            gate_off = 8
            wide = torch.zeros((st.n_rows, g.shape[1] + 16), dtype=TD[self.dtype], device="cuda")
            wide[:, gate_off:gate_off + g.shape[1]] = dev(g, TD[self.dtype])
        out = torch.full((st.n_rows, H * vd), 77.0, dtype=TD[self.dtype], device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        bt = ints(self.table if table is None else table)
        tail = (H, G, d, vd, self.ps, self.scale, self.window, 0, dev(self.talk) if self.talk is not None else None,
                dev(self.sinks) if self.sinks is not None else None, wide, gate_off, self.gate_kind == "head", 1.0)
        if kernel == "plain":
            ops.talk_attention_plain(qd, self.pool, 1, out, st.positions, st.seq, st.slots, bt, *tail, status=status)
        elif kernel == "items":
            items = ints(list(range(st.n))[::-1] + [-1, -1])
            ops.talk_attention_plain(qd, self.pool, 1, out, st.positions, st.seq, st.slots, bt, *tail, status=status,
                                     items=items, n_items=st.n + 2)
        elif kernel == "single":
            items = ints(list(range(st.n))[::-1] + [-1, -1])
            cap = max(s + n for _, s, n in entries)
            cap = min(cap, self.window) if self.window else cap
            cap = (cap + 7) // 8 * 8 + 8                 # a recorded step's bound is a padded one
            scratch = torch.full((ops.talk_attention_single_scratch(st.n + 2, H, cap),), 1e9, device="cuda")
            ops.talk_attention_single(qd, self.pool, 1, out, st.positions, st.seq, st.slots, bt, *tail, scratch, cap,
                                      status=status, items=items, n_items=st.n + 2)
        else:
            rows = ops.attention_prefill_tile_rows()
            tiles = [(k, off) for k, (_, _, n) in enumerate(entries) for off in range(0, n, rows)]
            tiles = tiles[::-1] + [(0, 1 << 24)]
            ops.talk_attention_tiles(qd, self.pool, 1, out, ints(tiles), len(tiles), rows, st.q_start, st.start_pos,
                                     st.slots, bt, *tail, status=status)
        assert int(status.item()) == 0, (kernel, entries)
        o = out.float().cpu().numpy()
        assert np.all(o[st.n:] == 77.0)
        res, at = {}, 0
        for i, s, n in entries:
            res[i] = o[at:at + n]
            at += n
        return res


def talk_kernels(dtype, H, G, d, vd):
    from swifttransformer_b200 import ops
    probe, out = torch.zeros(1, dtype=torch.bfloat16, device="cuda"), ["plain", "items"]
    if dtype == "bfloat16" and ops.talk_attention_tiles_applies(probe, H, G, d, vd):
        out.append("tiles")
    if dtype == "bfloat16" and ops.talk_attention_single_applies(probe, H, G, d, vd, 512):
        out.append("single")
    return out


TALK_SHAPES = [  # H, G, d, vd, ps, window, talk, sinks, gate
    (6, 2, 16, 24, 8, 21, True, True, "head"),
    (4, 4, 32, 8, 16, 0, True, False, None),          # every head its own keys; all earlier keys; no extra term
    (8, 1, 64, 72, 4, 64, True, True, "head"),        # eight heads on one key/value head
    (3, 3, 12, 20, 16, 7, True, True, "element"),     # sizes only the plain kernel takes
    (16, 4, 40, 48, 32, 130, True, True, "head"),     # pages of 32; a window longer than a tile of queries
    (2, 1, 128, 128, 16, 100, False, True, "head"),   # no mixing matrix: the identity
    (1, 1, 8, 8, 8, 1, True, True, "head"),           # one head, a window of one key
    (32, 8, 64, 128, 16, 100, True, True, "head"),    # more heads than one block's registers hold: value rows cut in two
    (24, 4, 32, 64, 8, 40, True, True, "element"),    # two heads per warp of sixteen
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", TALK_SHAPES)
def test_mixed_heads_attention_whole_in_portions_decoded_and_batched(dtype, shape):
    H, G, d, vd, ps, window, talk, sinks, gate = shape
    lengths = [300, 1, 37]
    case = TalkCase(lengths, H, G, d, vd, ps, seed=H * d, dtype=dtype, window=window, talk=talk, sinks=sinks, gate=gate)
    case.write_pool()
    refs = [case.reference(i) for i in range(len(lengths))]
    scale = max(np.abs(r).max() for r in refs)
    tol = (2e-5 if dtype == "float32" else 2.5e-2) * scale
    for kernel in talk_kernels(dtype, H, G, d, vd):
        def close(got, i, s, what):
            err = np.abs(got - refs[i][s:s + len(got)]).max(axis=1)
            assert err.max() < tol, (kernel, what, i, s + int(np.argmax(err)), float(err.max()), scale)
        alone = {}
        for i, n in enumerate(lengths):
            alone[i] = case.run([(i, 0, n)], kernel)[i]
            close(alone[i], i, 0, "whole")
        got = case.run([(i, 0, n) for i, n in enumerate(lengths)], kernel, pad_tokens=3)
        for i in got:
            close(got[i], i, 0, "batch")
            assert np.abs(got[i] - alone[i]).max() < tol
        cuts = [portions(n, (5, 2, 33, 1, 1, 130, 17, 2, 64)) for n in lengths]
        for k in range(max(len(c) for c in cuts)):
            entries = [(i, *cuts[i][k]) for i in range(len(lengths)) if k < len(cuts[i])]
            table = case.table
            for i, s, n in entries:
                table = np.where(np.arange(len(table))[:, None] == case.slot[i], case.drop_pages_out_of_sight(i, s), table)
            got = case.run(entries, kernel, table=table)
            for i, s, n in entries:
                close(got[i], i, s, "portion")
        if kernel != "tiles":
            for s in list(range(0, 12)) + list(range(lengths[0] - 40, lengths[0])):
                close(case.run([(0, s, 1)], kernel, table=case.drop_pages_out_of_sight(0, s))[0], 0, s, "decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ps,window", [(16, 0), (16, 50), (4, 64), (8, 129)])
def test_one_key_decides_at_every_edge_of_the_window(dtype, ps, window):
    """A key made to stand out: a query's result is that key's value exactly when the window lets the query see it:
    far back, on either side of a page border, the first tokens, just inside and just outside the window; in a
    portion of a prompt and decoded alone.  The key after the query never.  (No mixing here: the mask is the point.)"""
    H, G, d, vd, n = 4, 2, 16, 8, 420
    edges = {0, 1, ps - 1, ps, 3 * ps - 1, 3 * ps, 200, n - 2, n - 1}
    for kernel in talk_kernels(dtype, H, G, d, vd):
        for key in sorted(edges):
            case = TalkCase([n], H, G, d, vd, ps, seed=key, dtype=dtype, window=window, talk=False, sinks=True, gate=None)
            case.sinks[:] = -30.0
            loud = bf16_round(np.sign(case.k[0][key]) * 8.0)
            case.k[0][key] = loud
            queries = {key - 1, key, key + 1, key + ps, n - 1}
            if window:
                queries |= {key + window - 2, key + window - 1, key + window, key + window + 1}
            queries = sorted(t for t in queries if 0 <= t < n)
            for t in queries:
                case.q[0][t] = np.repeat(loud, H // G, axis=0) * 4.0
            case.write_pool()
            for t in queries:
                sees = key <= t and (not window or t - key < window)
                for form, (s, cnt) in (("portion", (max(0, t - 20), min(21, t + 1))), ("decoded", (t, 1))):
                    if form == "decoded" and kernel == "tiles":
                        continue
                    got = case.run([(0, s, cnt)], kernel, table=case.drop_pages_out_of_sight(0, s))[0][t - s]
                    want = np.repeat(case.v[0][key], H // G, axis=0)
                    if sees:
                        assert np.abs(got.reshape(H, vd) - want).max() < 0.05, (kernel, form, key, t)
                    else:
                        assert np.abs(got.reshape(H, vd) - want).max() > 0.3, (kernel, form, key, t)


@pytest.mark.parametrize("dtype", DTYPES)
def test_extra_term_is_per_head_unmixed_and_the_matrix_moves_weights_between_heads(dtype):
    """All scores zero: head b's weights are uniform over the seen keys with the share of its own extra term taken
    off.  A mixing matrix that hands head 0 the weights of head 1 (and nothing of its own) gives head 0 the sum of
    ITS OWN group's values under head 1's denominator."""
    H, G, d, vd, ps, window = 4, 2, 8, 16, 8, 12
    case = TalkCase([40], H, G, d, vd, ps, seed=3, dtype=dtype, window=window, talk=True, sinks=True, gate=None)
    case.q[0][:] = 0.0
    case.sinks[:] = np.log([1.0, 5.0, 0.25, 2.0])
    T = np.zeros((H, H))
    T[0, 3], T[1, 1], T[2, 0], T[3, 2] = 1.0, 1.0, 2.0, -1.0
    case.talk = T
    case.write_pool()
    extra = np.exp(case.sinks)
    for kernel in talk_kernels(dtype, H, G, d, vd):
        got = case.run([(0, 0, 40)], kernel)[0].reshape(40, H, vd)
        for t in (0, 1, 11, 12, 13, 39):
            seen = [j for j in range(t + 1) if t - j < window]
            for a, (b, c) in enumerate(((3, 1.0), (1, 1.0), (0, 2.0), (2, -1.0))):
                ref = c * case.v[0][seen, a // 2].sum(axis=0) / (len(seen) + extra[b])
                assert np.abs(got[t, a] - ref).max() < 2e-2, (kernel, t, a)


def test_prepare_norms_queries_and_keys_after_the_rotation():
    """The fused projection's columns q | k | v with biases: rotation of part of each head, then every query and key
    head divided by its root mean square; values as they are; pages as the block table names them."""
    from swifttransformer_b200 import ops
    for dtype in DTYPES:
        for H, G, d, vd, rot_dims, base, ps, eps in ((3, 1, 12, 5, 8, 50.0, 4, 1e-2), (4, 2, 16, 24, 16, 1e4, 8, 1e-6),
                                                     (2, 2, 40, 10, 0, 1.0, 16, 1e-5)):
            rng = np.random.default_rng(H + d)
            n, start, slot = 21, 9, 2
            qw, kw, vw = H * d, G * d, G * vd
            proj = bf16_round(rng.normal(size=(n, qw + kw + vw + 7)))
            bias = rng.normal(size=qw + kw + vw + 7).astype(np.float32).astype(np.float64)
            st = Step([(slot, start, n)], pad_tokens=2)
            n_pages = (start + n + ps - 1) // ps
            table = np.full((3, n_pages + 1), -1, dtype=np.int32)
            table[slot, :n_pages] = np.arange(n_pages)[::-1] + 1
            pool = torch.full((n_pages + 2, 2, G * ps * (d + vd)), 9.0, dtype=TD[dtype], device="cuda")
            q_out = torch.full((st.n_rows, qw), 7.0, dtype=TD[dtype], device="cuda")
            rows = dev(np.concatenate([proj, np.zeros((2, proj.shape[1]))]), TD[dtype])
            half = rot_dims // 2
            inv_freq = dev(base ** (-2.0 * np.arange(half) / max(rot_dims, 1))) if rot_dims else None
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            ops.gqa_prepare(rows, 0, qw, qw + kw, dev(bias), inv_freq, rot_dims, 0.0, 1, q_out, pool, 1, st.positions,
                            st.seq, st.slots, ints(table), H, G, d, vd, ps, status, norm_eps=eps)
            assert int(status.item()) == 0
            pos = np.arange(start, start + n)
            x = proj + bias
            q = pn.rms_unit(pn.rotate_halves(x[:, :qw].reshape(n, H, d), pos, rot_dims, base), eps)
            k = pn.rms_unit(pn.rotate_halves(x[:, qw:qw + kw].reshape(n, G, d), pos, rot_dims, base), eps)
            v = x[:, qw + kw:qw + kw + vw].reshape(n, G, vd)
            tol = 1e-5 if dtype == "float32" else 2e-2
            got_q = q_out.float().cpu().numpy()
            assert np.abs(got_q[:n].reshape(n, H, d) - q).max() < tol * np.abs(q).max()
            assert np.all(got_q[n:] == 7.0)
            pages = pool.float().cpu().numpy()
            assert np.all(pages[:, 0] == 9.0) and np.all(pages[0] == 9.0) and np.all(pages[-1] == 9.0)
            keys = pages[:, 1, :G * ps * d].reshape(-1, G, ps, d)
            vals = pages[:, 1, G * ps * d:].reshape(-1, G, ps, vd)
            for t, p in enumerate(pos):
                page = table[slot, p // ps]
                assert np.abs(keys[page, :, p % ps] - k[t]).max() < tol * np.abs(k).max()
                assert np.abs(vals[page, :, p % ps] - v[t]).max() < tol * np.abs(v).max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_grouped_attention_with_a_sink_per_head(dtype):
    """The kernels of the plain grouped attention with a learned logit per head in the denominator: all scores zero,
    so head a's result is the mean of the seen values scaled by n / (n + exp(sink_a))."""
    from swifttransformer_b200 import ops
    H, G, d, vd, ps, window, n = 4, 2, 16, 8, 8, 12, 40
    rng = np.random.default_rng(8)
    v = bf16_round(rng.normal(size=(n, G, vd)))
    sinks = np.log([1.0, 5.0, 0.25, 2.0])
    n_pages = n // ps
    keys, vals = np.zeros((n_pages, G, ps, d)), v.reshape(n_pages, ps, G, vd).transpose(0, 2, 1, 3)
    pool = dev(np.concatenate([keys.reshape(n_pages, 1, -1), vals.reshape(n_pages, 1, -1)], axis=2), TD[dtype])
    st = Step([(0, 0, n)])
    q = torch.zeros((n, H * d), dtype=TD[dtype], device="cuda")
    table = ints(np.arange(n_pages)[None])
    kernels = ["plain"] + (["tiles", "single"] if dtype == "bfloat16" else [])
    for kernel in kernels:
        out = torch.empty((n, H * vd), dtype=TD[dtype], device="cuda")
        consts = (H, G, d, vd, ps, 0.3, window, 0, dev(sinks), None, 0, 1.0)
        if kernel == "plain":
            ops.gqa_attention_plain(q, pool, 0, out, st.positions, st.seq, st.slots, table, *consts)
        elif kernel == "single":
            ops.gqa_attention_single(q, pool, 0, out, st.positions, st.seq, st.slots, table, *consts)
        else:
            ops.gqa_attention_tiles(q, pool, 0, out, ints([(0, 0)]), 1, ops.attention_prefill_tile_rows(), st.q_start,
                                    st.start_pos, st.slots, table, *consts)
        got = out.float().cpu().numpy().reshape(n, H, vd)
        for t in (0, 5, 11, 12, 30, 39):
            seen = [j for j in range(t + 1) if t - j < window]
            for a in range(H):
                ref = v[seen, a // 2].sum(axis=0) / (len(seen) + np.exp(sinks[a]))
                assert np.abs(got[t, a] - ref).max() < 2e-2, (kernel, t, a)


# ------------------------------------------------------------------------------------------ the gated delta rule
def delta_case(H, G, d, dv, taps, seed, T, slow_decay=False):
    rng = np.random.default_rng(seed)
    W = 24
    w = {"q": rng.normal(size=(G * d, W)) * 0.4, "k": rng.normal(size=(G * d, W)) * 0.4,
         "v": rng.normal(size=(H * dv, W)) * 0.4, "b": rng.normal(size=(H, W)) * 0.4, "a": rng.normal(size=(H, W)) * 0.4,
         "g": rng.normal(size=(H * dv, W)) * 0.4, "o": np.eye(H * dv),
         "q.conv": rng.normal(size=(G * d, taps)) * 0.6, "k.conv": rng.normal(size=(G * d, taps)) * 0.6,
         "v.conv": rng.normal(size=(H * dv, taps)) * 0.6, "A_log": rng.normal(size=H) * 0.5 - (5.0 if slow_decay else 0.0),
         "dt_bias": rng.normal(size=H) * 0.5, "norm": 1 + 0.1 * rng.normal(size=dv)}
    w = {k: bf16_round(v) for k, v in w.items()}
    return w, bf16_round(rng.normal(size=(T, W)))


def run_delta(w, h, H, G, d, dv, taps, dtype, cuts, slot=1, n_slots=3, eps=1e-5):
    """The mixer's kernels over the rows of h cut into steps (start, n); -> the heads' outputs [T, H * dv]."""
    from swifttransformer_b200 import ops
    channels = 2 * G * d + H * dv
    w_in = np.concatenate([w["q"], w["k"], w["v"], w["b"], w["a"], w["g"]])
    conv_w = dev(np.concatenate([w["q.conv"], w["k.conv"], w["v.conv"]]))
    tails = torch.zeros((n_slots, taps - 1, channels), dtype=torch.float32, device="cuda")
    S = torch.zeros((n_slots, H, d, dv), dtype=torch.float32, device="cuda")
    outs = []
    for start, n in cuts:
        st = Step([(slot, start, n)], pad_tokens=1, pad_requests=1)
        rows = np.concatenate([h[start:start + n] @ w_in.T, np.zeros((1, w_in.shape[0]))])
        proj = dev(rows)
        out = torch.zeros((st.n_rows, H * dv), dtype=TD[dtype], device="cuda")
        scratch = torch.empty(ops.delta_rule_scratch(st.n_rows, H, G, d, dv), dtype=torch.float32, device="cuda")
        single = n == 1
        ops.delta_rule(proj, channels, channels + H, channels + 2 * H, conv_w, tails, None, dev(w["A_log"]),
                       dev(w["dt_bias"]), None, dev(w["norm"]), eps, 1.0, S, True, single, scratch, out, st.positions,
                       st.seq, st.q_start, st.slots, st.n_seqs, H, G, d, dv, gate_silu=True)
        if taps > 1 and not single:
            ops.conv_state_update(proj, channels, tails, st.positions, st.q_start, st.slots, st.n_seqs)
        outs.append(out.float().cpu().numpy()[:n])
    assert float(S[0].abs().max()) == 0.0 and (taps == 1 or float(tails[0].abs().max()) == 0.0)     # the padding request's slot
    return np.concatenate(outs)


DELTA_SHAPES = [(4, 2, 16, 8, 4), (3, 3, 40, 24, 2), (2, 1, 130, 12, 1), (6, 1, 8, 64, 8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_delta_rule_with_a_decay_per_head_in_portions_and_token_by_token(dtype, shape):
    H, G, d, dv, taps = shape
    T = 70
    w, h = delta_case(H, G, d, dv, taps, seed=H * d, T=T)
    ref = pn.gated_delta(h, w, "", dict(heads=H, kv_heads=G, dim=d, vdim=dv), 1e-5)
    tol = (3e-5 if dtype == "float32" else 1.5e-2) * np.abs(ref).max()
    for cuts in ([(0, T)], portions(T, (5, 2, 1, 33, 1, 2, 9)), [(t, 1) for t in range(T)]):
        got = run_delta(w, h, H, G, d, dv, taps, dtype, cuts)
        err = np.abs(got - ref).max(axis=1)
        assert err.max() < tol, (cuts[:3], int(np.argmax(err)), float(err.max()))


def test_delta_rule_remembers_a_far_token_under_a_slow_decay():
    """A value written at token 3 is read out by a matching query 400 tokens later (through portions and single
    steps); with the state lost or reset on the way the read-out would be that of an empty state."""
    H, G, d, dv, taps, T = 2, 1, 16, 8, 2, 420
    w, h = delta_case(H, G, d, dv, taps, seed=5, T=T, slow_decay=True)
    h[4:T - 1] *= 0.02
    h[T - 1] = h[3]
    ref = pn.gated_delta(h, w, "", dict(heads=H, kv_heads=G, dim=d, vdim=dv), 1e-5)
    blank = pn.gated_delta(h[4:], w, "", dict(heads=H, kv_heads=G, dim=d, vdim=dv), 1e-5)
    assert np.abs(ref[-1] - blank[-1]).max() > 0.1 * np.abs(ref[-1]).max()
    got = run_delta(w, h, H, G, d, dv, taps, "float32", portions(T, (150, 1, 1, 2, 97)))
    assert np.abs(got[-1] - ref[-1]).max() < 1e-4 * np.abs(ref).max()


# ------------------------------------------------------------------------------------------ routed clamped experts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,limit", [(5, 3, 24, 1.0), (8, 1, 64, 2.5), (2, 2, 16, 0.3)])
def test_clamped_experts_with_renormalised_weights(dtype, E, top, ff, limit):
    from swifttransformer_b200.parts.base import FEED_FORWARDS
    rng = np.random.default_rng(E * ff)
    W, T = 40, 33
    w = {"router": bf16_round(rng.normal(size=(E, W)) * 1.5)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = bf16_round(rng.normal(size=(ff, W)) * 0.5), bf16_round(rng.normal(size=(ff, W)) * 0.5)
        w[f"e{e}.down"] = bf16_round(rng.normal(size=(W, ff)) * 0.3)
    h = bf16_round(rng.normal(size=(T, W)))
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    ref = pn.experts_ff(h, w, "", mlp)
    part = FEED_FORWARDS.build("routed_experts", hidden=W, inner=ff, num_experts=E, top=top, activation="none",
                               expert_names=[{k: f"e{e}.{k}" for k in ("gate", "up", "down")} for e in range(E)],
                               router_name="router", renormalise=True, limit=limit, alpha=1.702, shift=1.0)
    part.bind({k: dev(v, torch.float32 if k == "router" else TD[dtype]) for k, v in w.items()})

    class Ctx:
        positions = ints(list(range(T)) + [-1])
    rows = dev(np.concatenate([h, np.zeros((1, W))]), TD[dtype])
    got = part.forward(rows, Ctx).value.float().cpu().numpy()[:T]
    tol = (2e-5 if dtype == "float32" else 2e-2) * np.abs(ref).max()
    assert np.abs(got - ref).max() < tol


# ------------------------------------------------------------------------------------------ whole models
def left(heads, kv, dim, vdim, scale, size, dims, base):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if dims:
        m["rot"] = {"dims": dims, "base": base}
    return m


def right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def pair(l, r, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def attn(heads, kv, dim, vdim, scale, size, dims, base, mlp):
    return {"type": "attention", "mixer": left(heads, kv, dim, vdim, scale, size, dims, base), "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


CONFIGS = {
    # sizes that are multiples of nothing; attention first; three streams; a loop over two layers, twice; small
    # windows that pass over prompts and decoded tokens; a layer without feed-forward
    "mix": dict(cfg=dict(architecture="Nafelix", vocab=300, width=44, streams=3, norm={"eps": 1e-5}, canon={"taps": 2},
                         loop={"start": 1, "stop": 3, "times": 2}, layers=[
        attn(4, 2, 12, 7, 0.25, 9, 4, 100.0, dense(40)),
        pair(left(4, 2, 10, 12, 0.3, 12, 4, 100.0), right(2, 1, 9, 10, 3), moe(5, 3, 24, 1.0)),
        pair(left(3, 3, 6, 5, 0.4, 5, 6, 10.0), right(3, 3, 5, 7, 2), None),
        attn(6, 1, 6, 10, 0.3, 33, 2, 7.0, moe(3, 1, 16, 0.5))]), seed=31, std=0.1, page_size=8),
    # sizes that the tensor-core kernels take; two streams; five taps; no loop; a window longer than a tile of queries
    "fast": dict(cfg=dict(architecture="Nafelix", vocab=200, width=64, streams=2, norm={"eps": 3e-6}, canon={"taps": 5},
                          layers=[
        pair(left(8, 2, 32, 16, 0.18, 40, 16, 1e4), right(4, 2, 16, 16, 4), moe(4, 2, 32, 2.5)),
        attn(4, 1, 16, 24, 0.25, 130, 16, 3e5, dense(48)),
        pair(left(4, 4, 16, 32, 0.3, 150, 8, 50.0), right(2, 2, 32, 8, 2), dense(64)),
        attn(8, 8, 8, 8, 0.35, 17, 8, 9.0, moe(8, 2, 16, 1.5))]), seed=32, std=0.12, page_size=16),
    # one stream, no input convolutions, a loop that runs once, one head, a window of one key, an attention without
    # window and without rotation, one expert
    "lone": dict(cfg=dict(architecture="Nafelix", vocab=64, width=20, streams=1, norm={"eps": 1e-4},
                          loop={"start": 0, "stop": 1, "times": 1}, layers=[
        pair(left(1, 1, 4, 3, 0.5, 1, 2, 3.0), right(1, 1, 3, 4, 1), moe(1, 1, 8, 0.7)),
        attn(3, 1, 4, 6, 0.5, 0, 0, 1.0, None),
        pair(left(3, 1, 4, 6, 0.5, 1000, 4, 50.0), right(2, 1, 6, 3, 5), dense(16))]), seed=33, std=0.25, page_size=4),
}


@pytest.fixture(scope="module")
def nafelix_dirs(tmp_path_factory):
    return make_model_dirs(tmp_path_factory.mktemp("nafelix"))


def make_model_dirs(root):
    """Model folders with random weights.  The decays' logarithms are lowered, so that the recurrent state remembers
    for hundreds of tokens and a lost or mixed-up state shows; routers and sinks are made loud; biases are as large
    as the weights' products; the streams' coefficients are a perturbed identity, so that no copy dies out and every
    one of them matters."""
    from swifttransformer_b200.config import NafelixConfig, save_config
    from swifttransformer_b200.models import build_model_def
    from swifttransformer_b200.weights.random_init import random_tensors
    from swifttransformer_b200.weights.safetensors_io import write_safetensors
    out = {}
    for name, c in CONFIGS.items():
        cfg = NafelixConfig.from_dict(c["cfg"])
        path = str(root / name)
        save_config(cfg, path)
        n, tensors = cfg.streams, []
        for s, t in random_tensors(build_model_def(cfg).param_specs(), c["seed"], c["std"], "cpu"):
            f = t.float()
            if s.name.endswith(".A_log"):
                f = f - 4.0
            elif s.name.endswith(".router"):
                f = f * 6
            elif s.name.endswith((".sink", ".act")):
                f = f / c["std"] * 1.5
            elif s.name.endswith(".b") and t.dim() == 1:
                f = f * 3
            elif s.name.endswith(".talk"):
                f = torch.eye(t.shape[0]) + f / c["std"] * 0.3
            elif s.name.endswith((".hc1.in", ".hc2.in")):
                f = 1.0 / n + f / c["std"] * 0.1
            elif s.name.endswith((".hc1.out", ".hc2.out")):
                f = 1.0 + f / c["std"] * 0.15
            elif s.name.endswith((".hc1.mix", ".hc2.mix")):
                f = torch.eye(n) + f / c["std"] * 0.1
            elif s.name.endswith((".canon1", ".canon2")):
                f = f / c["std"] * 0.3
            tensors.append((s.name, f.to(torch.bfloat16)))
        write_safetensors(os.path.join(path, "model.safetensors"), tensors)
        out[name] = path
    return out


_PLAIN = {}


def plain_logits(model_dir, tokens):
    key = (model_dir, tuple(tokens))
    if key not in _PLAIN:
        if model_dir not in _PLAIN:
            _PLAIN[model_dir] = pn.load_model(model_dir)
        cfg, w = _PLAIN[model_dir]
        _PLAIN[key] = pn.forward(cfg, w, tokens)
    return _PLAIN[key]


def requests_for(name, lengths=(210, 1, 23, 97, 64)):
    vocab = CONFIGS[name]["cfg"]["vocab"]
    return {f"r{i}": helpers.random_tokens(vocab, n, seed=10 * i + len(name)) for i, n in enumerate(lengths)}


def compare(model_dir, reqs, got, dtype, what):
    """float32: every position within rounding.  bfloat16: rounding of the activations can hand a token to another
    expert where two scores nearly tie (a request of a single token may be such a token), so over all requests of a
    run a few positions may lie further off; most must be close and none wild."""
    tol = {"float32": 3e-5, "bfloat16": 5e-2}[dtype]
    errs = []
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        assert got[rid].shape == ref.shape, (what, rid)
        scale = np.abs(ref).max()
        if dtype == "float32":
            bad = helpers.first_bad(got[rid], ref, tol * scale)
            assert bad is None, (f"{what}/{dtype}: request {rid} first differs at position {bad[0]} of {len(toks)} by "
                                 f"{bad[1]:.3e} of {scale:.3e}")
        errs.append(np.abs(got[rid] - ref).max(axis=1) / scale)
    err = np.concatenate(errs)
    if dtype == "bfloat16":
        assert np.median(err) < tol / 2 and (err > tol).mean() <= 0.1 and err.max() < 10 * tol, \
            f"{what}/{dtype}: median {np.median(err):.3e}, over {(err > tol).mean():.3f}, worst {err.max():.3e} at {int(np.argmax(err))}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("schedule", ["whole", "decode", "portions", "mixed"])
def test_replay_matches_plain(nafelix_dirs, name, dtype, schedule):
    from swifttransformer_b200.engine.replay import TraceSession
    reqs = requests_for(name)
    steps = {"whole": helpers.trace_whole, "decode": lambda r: helpers.trace_decode_tail(r, tail=60),
             "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, seed=1, max_live=3)}[schedule](reqs)
    need = helpers.live_token_need(steps)
    s = TraceSession(nafelix_dirs[name], dtype, need, page_size=CONFIGS[name]["page_size"], max_requests=3)
    got = helpers.replay(s, steps)
    compare(nafelix_dirs[name], reqs, got, dtype, f"{name}/{schedule}")
    s.cache.check()
    assert all(g.pool.num_held == 0 for g in s.cache.groups)


def test_residual_stream_after_every_layer_run(nafelix_dirs):
    """Layer run by layer run (a looped layer counts every time): the sum of the streams."""
    from swifttransformer_b200.engine.replay import TraceSession
    for name in CONFIGS:
        toks = helpers.random_tokens(CONFIGS[name]["cfg"]["vocab"], 29, seed=5)
        s = TraceSession(nafelix_dirs[name], "float32", 64, page_size=CONFIGS[name]["page_size"], max_requests=1)
        s.runner.use_cuda_graphs = False
        got = []
        s.model.after_layer = lambda i, stream: got.append(stream.x.cpu().numpy().copy())
        s.run_step([dict(id="a", tokens=toks, want=[28])], ["a"])
        cfg, w = pn.load_model(nafelix_dirs[name])
        _, ref = pn.forward(cfg, w, toks, return_layers=True)
        assert len(got) == len(ref) == len(pn.layer_runs(cfg))
        for i in range(len(ref)):
            assert np.abs(got[i] - ref[i]).max() < 2e-5 * np.abs(ref[i]).max(), (name, i)


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_and_eager_steps_agree(nafelix_dirs, dtype):
    from swifttransformer_b200.engine.replay import TraceSession
    reqs = requests_for("fast", lengths=(70, 9))
    steps = helpers.trace_mixed(reqs, seed=2, max_live=2)
    outs = []
    for graphs in (True, False):
        s = TraceSession(nafelix_dirs["fast"], dtype, helpers.live_token_need(steps), max_requests=2)
        s.runner.use_cuda_graphs = graphs
        outs.append(helpers.replay(s, steps))
        assert (s.runner.graph_steps + s.runner.padded_graph_steps > 0) == graphs
    for rid in reqs:
        tol = 1e-5 if dtype == "float32" else 3e-2
        err = np.abs(outs[0][rid] - outs[1][rid]).max(axis=1) / np.abs(outs[1][rid]).max()
        assert err.max() < tol, (rid, int(np.argmax(err)), float(err.max()))


@pytest.mark.parametrize("name", ["mix", "fast"])
def test_long_decoding_with_pages_and_slots_used_again(nafelix_dirs, name):
    """Three requests after one another through the same single slot and a pool that holds only one of them, each
    decoded token by token for 300 steps after a short prompt: the windows pass over decoded tokens, their pages come
    back, and the next request starts from zero states (the recurrence's, and every convolution's) in the slot the
    last one left."""
    from swifttransformer_b200.engine.replay import TraceSession
    ps = CONFIGS[name]["page_size"]
    s = TraceSession(nafelix_dirs[name], "float32", 384, page_size=ps, max_requests=1)
    for k in range(3):
        toks = helpers.random_tokens(CONFIGS[name]["cfg"]["vocab"], 330, seed=40 + k)
        rows = [s.run_step([dict(id=k, tokens=toks[:30], want=list(range(30)))]).cpu().numpy().copy()]
        for t in range(30, 330):
            rows.append(s.run_step([dict(id=k, tokens=[toks[t]], want=[0])], [k] if t == 329 else []).cpu().numpy().copy())
        s.check()
        ref = plain_logits(nafelix_dirs[name], toks)
        bad = helpers.first_bad(np.concatenate(rows), ref, 3e-5 * np.abs(ref).max())
        assert bad is None, (k, bad)
    assert all(g.pool.num_held == 0 for g in s.cache.groups)


def test_windows_give_their_pages_back(nafelix_dirs):
    """A model whose every attention has a window holds, however long the request grows, only the window's pages."""
    from swifttransformer_b200.engine.replay import TraceSession
    s = TraceSession(nafelix_dirs["mix"], "float32", 2048, page_size=8, max_requests=1)
    toks = helpers.random_tokens(300, 600, seed=9)
    s.run_step([dict(id=0, tokens=toks[:500], want=[])])
    assert max(g.pool.num_held for g in s.cache.groups) <= 33 // 8 + 2
    got = s.run_step([dict(id=0, tokens=toks[500:], want=[99])]).cpu().numpy()
    ref = plain_logits(nafelix_dirs["mix"], toks)
    assert np.abs(got[0] - ref[599]).max() < 3e-5 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "fast"])
def test_greedy_generation_through_the_engine(nafelix_dirs, name, dtype):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.sampling.sampler import SamplingParams
    vocab = CONFIGS[name]["cfg"]["vocab"]
    prompts = [helpers.random_tokens(vocab, n, seed=n) for n in (5, 31, 1, 18, 44, 9)]
    eng = LLMEngine(nafelix_dirs[name], dtype=dtype, page_size=CONFIGS[name]["page_size"], num_pages=24,
                    max_num_seqs=3, max_batch_tokens=48, chunk_size=20, max_seq_len=256)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0))
    cfg, w = pn.load_model(nafelix_dirs[name])
    for prompt, out in zip(prompts, outs):
        toks = list(prompt)
        tokens = list(out.output if hasattr(out, "output") else out)
        assert len(tokens) == 12
        for k, tok in enumerate(tokens):
            logits = pn.forward(cfg, w, toks)[-1]
            best = int(np.argmax(logits))
            if tok != best:
                gap = logits[best] - logits[tok]
                assert dtype == "bfloat16" and gap < 0.08 * np.abs(logits).max(), (name, k, tok, best, gap)
            toks.append(tok)


# ------------------------------------------------------------------------------------------ the programs
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_run_gpt_takes_a_nafelix_folder(nafelix_dirs, tmp_path):
    import subprocess
    import sys
    vocab = CONFIGS["mix"]["cfg"]["vocab"]
    prompts = [helpers.random_tokens(vocab, n, 70 + n) for n in (6, 21)]
    inp = tmp_path / "in.txt"
    inp.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_gpt"), nafelix_dirs["mix"], "any", "fp32", str(inp),
                        "--max_decoding_step", "5", "--num_total_blocks", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = pn.load_model(nafelix_dirs["mix"])
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 2
    for line, p in zip(lines, prompts):
        got = [int(t) for t in line.split(")")[1].split("(")[0].split()]
        assert got == pn.greedy(cfg, w, p, 5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program_with_four_slots(nafelix_dirs, tmp_path, dtype):
    """bin/trace_run with its defaults (four request slots, pages of 16): six requests, at most four live, so slots and
    pages are handed out again; every wanted row against the plain implementation."""
    import subprocess
    import sys
    name = "fast"
    reqs = requests_for(name, lengths=(50, 1, 33, 170, 18, 40))
    steps = helpers.trace_mixed(reqs, seed=3, max_live=4)
    out = tmp_path / "out"
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", nafelix_dirs[name], "--dtype", dtype,
                          "--out", str(out), "--max-tokens", str(helpers.live_token_need(steps))],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    got = {rid: [] for rid in reqs}
    vocab = CONFIGS[name]["cfg"]["vocab"]
    for i, st in enumerate(steps):
        p.stdin.write(json.dumps(dict(st, step=i)) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {i}", p.stderr.read()[-2000:]
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in st["entries"]:
            got[e["id"]].append(arr[k:k + len(e["want"])])
            k += len(e["want"])
        assert k == len(arr)
    p.stdin.close()
    assert p.wait(timeout=120) == 0
    compare(nafelix_dirs[name], reqs, {rid: np.concatenate(v) for rid, v in got.items()}, dtype, "trace_run")
