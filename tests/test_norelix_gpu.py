"""The Norelix design on the GPU against the plain implementation (tests/plain_norelix.py).

Mechanisms alone (the kernels driven directly over a small paged cache and state slots, with inputs made so
that a single key or an edge decides the result), then whole models of several small configurations through
the trace replay (whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with
pages and slots used again) and through ``LLMEngine.generate``.
"""
from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_norelix as pn

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def bf16_round(a):
    """float64 array with values that bfloat16 holds exactly."""
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(torch.bfloat16).double().numpy()


class Step:
    """The index arrays of one step for given (slot, start, n) entries, as the step function lays them out,
    with padding tokens at position -1 and padding requests behind."""

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


# ------------------------------------------------------------------------------------------ the feed-forward's unit
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner,limit", [(37, 1.5), (256, 7.0), (64, 0.25)])
def test_gated_clamped_act(dtype, inner, limit):
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(inner)
    gu = bf16_round(rng.normal(size=(11, 2 * inner)) * 3)
    bias = rng.normal(size=2 * inner).astype(np.float32).astype(np.float64)
    out = ops.gated_clamped_act(dev(gu, TD[dtype]), dev(bias), limit, 1.702, 1.0).float().cpu().numpy()
    ref = pn.clamped_unit(gu[:, :inner] + bias[:inner], gu[:, inner:] + bias[inner:], limit)
    # both limits bite somewhere, or the case tests nothing
    assert (gu[:, :inner] + bias[:inner] > limit).any() and (np.abs(gu[:, inner:] + bias[inner:]) > limit).any()
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert np.all(np.abs(out - ref) <= tol * (1 + np.abs(ref)))


# ------------------------------------------------------------------------------------------ the gated delta rule
def delta_case(H, G, d, dv, taps, rank, seed, T, slow_decay=False):
    """Weights of one right-hand mixer with the output projection left out (identity), and its input rows."""
    rng = np.random.default_rng(seed)
    W = 48
    p = "m."
    w = {p + "q": rng.normal(size=(G * d, W)) * 0.3, p + "k": rng.normal(size=(G * d, W)) * 0.3,
         p + "v": rng.normal(size=(H * dv, W)) * 0.3, p + "b": rng.normal(size=(H, W)) * 0.3,
         p + "a1": rng.normal(size=(rank, W)) * 0.3, p + "a2": rng.normal(size=(H * d, rank)) * 0.5,
         p + "g1": rng.normal(size=(rank + 1, W)) * 0.3, p + "g2": rng.normal(size=(H * dv, rank + 1)) * 0.5,
         p + "A_log": rng.normal(size=H) - (6.0 if slow_decay else 0.5), p + "dt_bias": rng.normal(size=H * d) * 0.5,
         p + "norm": 1 + 0.2 * rng.normal(size=dv), p + "o": np.eye(H * dv)}
    for key, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
        w[p + key + ".conv"] = rng.normal(size=(rows, taps)) * 0.6
    w = {k: bf16_round(v) for k, v in w.items()}
    h = bf16_round(rng.normal(size=(T, W)))
    return w, h


def run_delta(w, h, H, G, d, dv, taps, dtype, cuts, slot=1, n_slots=3):
    """The mixer's kernels over the rows of one request cut into portions; returns (result, states, tails)."""
    from swifttransformer_b200 import ops
    p = "m."
    w_in = np.concatenate([w[p + k] for k in ("q", "k", "v", "b", "a1", "g1")])
    proj_all = (h @ w_in.T).astype(np.float32)
    C = 2 * G * d + H * dv
    ra = w[p + "a1"].shape[0]
    b_off, a_off, g_off = C, C + H, C + H + ra
    conv_w = dev(np.concatenate([w[p + k + ".conv"] for k in "qkv"]))
    state = torch.zeros((n_slots, H, d, dv), device="cuda")
    tails = torch.zeros((n_slots, taps - 1, C), device="cuda")
    state[0].fill_(3.0)
    tails[0].fill_(5.0)
    got = np.zeros((len(h), H * dv))
    for start, n in cuts:
        st = Step([(slot, start, n)], pad_tokens=2, pad_requests=1)
        rows = dev(np.concatenate([proj_all[start:start + n], np.full((2, proj_all.shape[1]), 7.0)]))
        out = torch.zeros((st.n_rows, H * dv), dtype=TD[dtype], device="cuda")
        single = n == 1
        scratch = torch.full((ops.delta_rule_scratch(st.n_rows, H, G, d, dv),), 9.0, device="cuda")
        ops.delta_rule(rows, b_off, a_off, g_off, conv_w, tails, dev(w[p + "a2"], TD[dtype]), dev(w[p + "A_log"]),
                       dev(w[p + "dt_bias"]), dev(w[p + "g2"], TD[dtype]), dev(w[p + "norm"]), 1e-5, 0.7, state, True,
                       single, scratch, out, st.positions, st.seq, st.q_start, st.slots, st.n_seqs, H, G, d, dv)
        if taps > 1 and not single:
            ops.conv_state_update(rows, C, tails, st.positions, st.q_start, st.slots, st.n_seqs)
        got[start:start + n] = out.float().cpu().numpy()[:n]
    assert torch.all(state[0] == 3.0) and torch.all(tails[0] == 5.0) and torch.all(state[2] == 0.0)
    return got, state, tails


DELTA_SHAPES = [  # H, G, d, dv, taps, rank
    (4, 2, 16, 24, 3, 5),
    (2, 2, 40, 72, 4, 8),
    (3, 1, 130, 20, 2, 3),        # a key size beyond 128: the wide layout of the recurrence
    (1, 1, 8, 136, 1, 4),         # no convolution at all
    (2, 1, 64, 48, 8, 16),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_delta_rule_in_portions_and_token_by_token(dtype, shape):
    H, G, d, dv, taps, rank = shape
    T = 70
    w, h = delta_case(H, G, d, dv, taps, rank, seed=H * 100 + d, T=T, slow_decay=True)
    mx = dict(heads=H, kv_heads=G, dim=d, vdim=dv, conv=taps)
    ref = 0.7 * pn.gated_delta(h, w, "m.", mx, 1e-5)
    tol = (3e-5 if dtype == "float32" else 2e-2) * np.abs(ref).max()
    for sizes in ((T,), (17, 2, 1, 1, 1, 30, 1, 1), (1,), (2,)):
        got, _, _ = run_delta(w, h, H, G, d, dv, taps, dtype, portions(T, sizes))
        err = np.abs(got - ref).max(axis=1)
        assert err.max() < tol, (sizes, int(np.argmax(err > tol)), float(err.max()))


@pytest.mark.parametrize("lanes", [8, 16])
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_delta_rule_with_every_layout_of_the_state(lanes, shape):
    from swifttransformer_b200 import ops
    H, G, d, dv, taps, rank = shape
    T = 45
    w, h = delta_case(H, G, d, dv, taps, rank, seed=H * 10 + d + lanes, T=T, slow_decay=True)
    ref = 0.7 * pn.gated_delta(h, w, "m.", dict(heads=H, kv_heads=G, dim=d, vdim=dv, conv=taps), 1e-5)
    ops.delta_rule_set_lanes(lanes)
    try:
        for sizes in ((T,), (9, 1, 1, 2, 30, 1, 1)):
            got, _, _ = run_delta(w, h, H, G, d, dv, taps, "float32", portions(T, sizes))
            assert np.abs(got - ref).max() < 3e-5 * np.abs(ref).max(), (lanes, sizes)
    finally:
        ops.delta_rule_set_lanes(0)


def test_delta_rule_remembers_a_far_token_and_forgets_with_decay():
    """One token writes a value along a key; fifty tokens later a query along that key reads it back when the
    decays are near one, and reads nothing when they are strong."""
    H, G, d, dv, taps, rank = 1, 1, 16, 8, 1, 2
    for slow in (True, False):
        w, h = delta_case(H, G, d, dv, taps, rank, seed=3, T=60, slow_decay=slow)
        if not slow:
            w["m.A_log"] = np.array([3.0])
        mx = dict(heads=H, kv_heads=G, dim=d, vdim=dv, conv=taps)
        ref = pn.gated_delta(h, w, "m.", mx, 1e-5)
        got, state, _ = run_delta(w, h, H, G, d, dv, taps, "float32", portions(60, (9, 1, 1, 30)))
        assert np.abs(got / 0.7 - ref).max() < 3e-5 * np.abs(ref).max()
        # the state of a strongly decaying head holds the last tokens only: its size tells the two apart
        norm = float(state[1].norm())
        assert (norm > 1.0) if slow else (norm < 2.5), (slow, norm)


def test_delta_rule_padding_request_leaves_slot_zero_alone():
    """A recorded decode step pads with requests of one token at position -1 whose slot index reads 0."""
    from swifttransformer_b200 import ops
    H, G, d, dv, taps, rank = 2, 1, 8, 8, 3, 2
    C = 2 * G * d + H * dv
    state = torch.full((2, H, d, dv), 5.0, device="cuda")
    tails = torch.full((2, taps - 1, C), 5.0, device="cuda")
    st = Step([], pad_tokens=2)
    st.q_start, st.slots, st.n_seqs = ints([0, 1, 2]), ints([0, 0]), 2
    rows = torch.ones((2, C + H + 2 * rank), device="cuda")
    out = torch.zeros((2, H * dv), device="cuda")
    scratch = torch.zeros(ops.delta_rule_scratch(2, H, G, d, dv), device="cuda")
    ops.delta_rule(rows, C, C + H, C + H + rank, torch.ones((C, taps), device="cuda"), tails,
                   torch.ones((H * d, rank), device="cuda"), torch.zeros(H, device="cuda"), torch.zeros(H * d, device="cuda"),
                   torch.ones((H * dv, rank), device="cuda"), torch.ones(dv, device="cuda"), 1e-5, 1.0, state, True, True,
                   scratch, out, st.positions, st.seq, st.q_start, st.slots, st.n_seqs, H, G, d, dv)
    assert torch.all(state == 5.0) and torch.all(tails == 5.0)


# ------------------------------------------------------------------------------------------ grouped attention
def test_prepare_adds_biases_rotates_scales_queries_and_fills_pages():
    """The fused projection's columns q | k | v | gate in wider rows: biases, the halves rotation on part of each head,
    the query temperature, and keys and values in the pages the block table names."""
    from swifttransformer_b200 import ops
    for dtype in DTYPES:
        for H, G, d, vd, rot_dims, base, temp, ps in ((3, 1, 12, 5, 8, 50.0, (0.4, 3), 4), (4, 2, 16, 24, 16, 1e4, None, 8),
                                                      (2, 2, 6, 10, 0, 1.0, (0.25, 1), 16)):
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
            ops.gqa_prepare(rows, 0, qw, qw + kw, dev(bias), inv_freq, rot_dims, temp[0] if temp else 0.0,
                            temp[1] if temp else 1, q_out, pool, 1, st.positions, st.seq, st.slots, ints(table), H, G, d, vd,
                            ps, status)
            assert int(status.item()) == 0
            pos = np.arange(start, start + n)
            x = proj + bias
            q, k = x[:, :qw].reshape(n, H, d), x[:, qw:qw + kw].reshape(n, G, d)
            if rot_dims:
                q, k = pn.rotate_halves(q, pos, rot_dims, base), pn.rotate_halves(k, pos, rot_dims, base)
            if temp:
                q = q * pn.temperature(pos, *temp)[:, None, None]
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
            # positions of the pages that the step did not bring stay as they were
            assert np.all(keys[table[slot, 0], :, :min(start, ps)] == 9.0)


class GqaCase:
    """Queries, keys, values and gate logits of a few requests; keys and values stand in a paged pool whose pages are
    dealt out of order and whose unused rows hold large numbers."""

    def __init__(self, lengths, H, G, d, vd, ps, seed, dtype, window=0, keep_first=0, sink=None, gate=True, out_scale=1.0):
        rng = np.random.default_rng(seed)
        self.H, self.G, self.d, self.vd, self.ps, self.dtype = H, G, d, vd, ps, dtype
        self.window, self.keep_first, self.sink, self.out_scale = window, keep_first, sink, out_scale
        self.lengths = list(lengths)
        self.q = [bf16_round(rng.normal(size=(n, H, d))) for n in lengths]
        self.k = [bf16_round(rng.normal(size=(n, G, d))) for n in lengths]
        self.v = [bf16_round(rng.normal(size=(n, G, vd))) for n in lengths]
        self.gate = [bf16_round(rng.normal(size=(n, H * vd))) for n in lengths] if gate else None
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

    def seen(self, n):
        return pn.seen_window(n, self.window, self.keep_first) if self.window else pn.seen_causal(n)

    def reference(self, i):
        n = self.lengths[i]
        seen = self.seen(n)
        out = np.zeros((n, self.H, self.vd))
        for a in range(self.H):
            g = a // (self.H // self.G)
            s = np.where(seen, self.q[i][:, a] @ self.k[i][:, g].T * self.scale, -np.inf)
            m = s.max(axis=1, keepdims=True)
            if self.sink is not None:
                m = np.maximum(m, self.sink)
            e = np.exp(s - m)
            den = e.sum(axis=1, keepdims=True) + (np.exp(self.sink - m) if self.sink is not None else 0.0)
            out[:, a] = (e / den) @ self.v[i][:, g] * self.out_scale
        out = out.reshape(n, -1)
        return out * pn.sigmoid(self.gate[i]) if self.gate is not None else out

    def drop_pages_out_of_sight(self, i, pos):
        """The block table as the cache manager leaves it when request i stands at position pos: pages wholly
        behind the window and past the kept first keys are gone."""
        table = self.table.copy()
        if self.window:
            lo = max(0, pos - self.window + 1)
            for page in range(lo // self.ps):
                if page * self.ps >= self.keep_first:
                    table[self.slot[i], page] = -1
        return table

    def run(self, entries, kernel, pad_tokens=0, table=None):
        """entries: (request, start, n).  kernel: 'plain', 'tiles' (every entry in tiles of query rows) or 'single'
        (every token an item).  -> {request: rows start..start+n-1 of the result}"""
        from swifttransformer_b200 import ops
        H, G, d, vd = self.H, self.G, self.d, self.vd
        st = Step([(self.slot[i], s, n) for i, s, n in entries], pad_tokens=pad_tokens)
        q = np.concatenate([self.q[i][s:s + n] for i, s, n in entries] + [np.full((pad_tokens, H, d), 50.0)])
        qd = dev(q.reshape(st.n_rows, -1), TD[self.dtype])
        wide, gate_off = None, 0
        if self.gate is not None:
            g = np.concatenate([self.gate[i][s:s + n] for i, s, n in entries] + [np.zeros((pad_tokens, H * vd))])
            gate_off = 8
            wide = torch.zeros((st.n_rows, H * vd + 16), dtype=TD[self.dtype], device="cuda")
            wide[:, gate_off:gate_off + H * vd] = dev(g, TD[self.dtype])
        out = torch.full((st.n_rows, H * vd), 77.0, dtype=TD[self.dtype], device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        bt = ints(self.table if table is None else table)
        consts = (H, G, d, vd, self.ps, self.scale, self.window, self.keep_first, self.sink, wide, gate_off, self.out_scale)
        if kernel == "plain":
            ops.gqa_attention_plain(qd, self.pool, 1, out, st.positions, st.seq, st.slots, bt, *consts, status=status)
        elif kernel == "single":
            items = ints(list(range(st.n))[::-1] + [-1, -1])
            ops.gqa_attention_single(qd, self.pool, 1, out, st.positions, st.seq, st.slots, bt, *consts, status=status,
                                     items=items, n_items=st.n + 2)
        else:
            rows = ops.attention_prefill_tile_rows()
            tiles = [(k, off) for k, (_, _, n) in enumerate(entries) for off in range(0, n, rows)]
            tiles = tiles[::-1] + [(0, 1 << 24)]
            ops.gqa_attention_tiles(qd, self.pool, 1, out, ints(tiles), len(tiles), rows, st.q_start, st.start_pos,
                                    st.slots, bt, *consts, status=status)
        assert int(status.item()) == 0, (kernel, entries)
        o = out.float().cpu().numpy()
        assert np.all(o[st.n:] == 77.0)
        res, at = {}, 0
        for i, s, n in entries:
            res[i] = o[at:at + n]
            at += n
        return res


def gqa_kernels(dtype, H, G, d, vd):
    from swifttransformer_b200 import ops
    if dtype == "bfloat16" and ops.gqa_attention_fast_applies(torch.zeros(1, dtype=torch.bfloat16, device="cuda"), H, G, d, vd):
        return ["plain", "tiles", "single"]
    return ["plain"]


GQA_SHAPES = [  # H, G, d, vd, ps, window, keep_first, sink, gate, out_scale
    (6, 2, 16, 24, 8, 21, 5, 0.0, False, 0.8),        # three query heads per key/value head, a sink, no gate
    (4, 4, 32, 8, 16, 0, 0, None, True, 1.0),         # every head its own keys; all earlier keys; gated
    (8, 1, 64, 72, 4, 64, 64, 1.5, True, 1.3),        # eight heads on one key/value head; window == kept == tile
    (2, 1, 128, 256, 16, 100, 1, None, False, 1.0),   # the largest sizes of the tensor-core kernel
    (3, 3, 12, 20, 16, 7, 0, -0.5, True, 0.5),        # sizes only the plain kernel takes; nothing kept
    (12, 4, 40, 48, 32, 130, 20, 0.0, True, 1.0),     # pages of 32; a window longer than a tile of queries
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", GQA_SHAPES)
def test_grouped_attention_whole_in_portions_decoded_and_batched(dtype, shape):
    H, G, d, vd, ps, window, keep, sink, gate, out_scale = shape
    lengths = [300, 1, 37]
    case = GqaCase(lengths, H, G, d, vd, ps, seed=H * d, dtype=dtype, window=window, keep_first=keep, sink=sink, gate=gate,
                   out_scale=out_scale)
    case.write_pool()
    refs = [case.reference(i) for i in range(len(lengths))]
    scale = max(np.abs(r).max() for r in refs)
    tol = (2e-5 if dtype == "float32" else 2e-2) * scale
    for kernel in gqa_kernels(dtype, H, G, d, vd):
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
        # portions of several sizes down to two tokens, two requests side by side; the pages behind the window are gone
        cuts = [portions(n, (5, 2, 33, 1, 1, 130, 17, 2, 64)) for n in lengths]
        for k in range(max(len(c) for c in cuts)):
            entries = [(i, *cuts[i][k]) for i in range(len(lengths)) if k < len(cuts[i])]
            table = case.table
            for i, s, n in entries:
                table = np.where(np.arange(len(table))[:, None] == case.slot[i], case.drop_pages_out_of_sight(i, s), table)
            got = case.run(entries, kernel, table=table)
            for i, s, n in entries:
                close(got[i], i, s, "portion")
        for s in list(range(0, 12)) + list(range(lengths[0] - 40, lengths[0])):
            close(case.run([(0, s, 1)], kernel, table=case.drop_pages_out_of_sight(0, s))[0], 0, s, "decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ps,window,keep", [(16, 0, 0), (16, 50, 6), (4, 64, 3), (8, 129, 17)])
def test_one_key_decides_at_every_edge(dtype, ps, window, keep):
    """A key made to stand out: a query's result is that key's value exactly when the mask lets the query see it: far
    back, on either side of a page border, the first token, just inside and just outside the window, the last kept
    first key and the one after it; in a portion of a prompt and decoded alone.  The key after the query never."""
    H, G, d, vd, n = 4, 2, 16, 8, 420
    edges = {0, 1, ps - 1, ps, 3 * ps - 1, 3 * ps, 200, n - 2, n - 1}
    if keep:
        edges |= {keep - 1, keep, keep + 1}
    for kernel in gqa_kernels(dtype, H, G, d, vd):
        for key in sorted(edges):
            case = GqaCase([n], H, G, d, vd, ps, seed=key, dtype=dtype, window=window, keep_first=keep, sink=-30.0, gate=False)
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
                sees = key <= t and (not window or t - key < window or key < keep)
                for form, (s, cnt) in (("portion", (max(0, t - 20), min(21, t + 1))), ("decoded", (t, 1))):
                    if form == "decoded" and kernel == "tiles":
                        continue
                    got = case.run([(0, s, cnt)], kernel, table=case.drop_pages_out_of_sight(0, s))[0][t - s]
                    got = got.reshape(H, vd)
                    want = np.repeat(case.v[0][key], H // G, axis=0)
                    if sees:
                        assert np.abs(got - want).max() < 0.05, (kernel, form, key, t)
                    else:
                        assert np.abs(got - want).max() > 0.3, (kernel, form, key, t)


@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_extra_term_takes_its_share_and_has_no_value(dtype):
    H, G, d, vd, ps = 3, 1, 8, 16, 8
    for sink, extra in ((0.0, 1.0), (np.log(5.0), 5.0), (None, 0.0)):
        case = GqaCase([40], H, G, d, vd, ps, seed=3, dtype=dtype, window=12, keep_first=2, sink=sink, gate=False)
        case.q[0][:] = 0.0                       # every score is 0: uniform weights over the seen keys
        case.write_pool()
        for kernel in gqa_kernels(dtype, H, G, d, vd):
            got = case.run([(0, 0, 40)], kernel)[0].reshape(40, H, vd)
            for t in (0, 1, 11, 12, 13, 14, 39):
                seen = [j for j in range(t + 1) if t - j < 12 or j < 2]
                ref = case.v[0][seen, 0].sum(axis=0) / (len(seen) + extra)
                assert np.abs(got[t] - ref[None]).max() < 2e-2, (kernel, sink, t)


# ------------------------------------------------------------------------------------------ whole models
def left(heads, kv, dim, vdim, scale, size, keep, dims, base):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask={"size": size, "keep_first": keep},
                rot={"dims": dims, "base": base})


def right(heads, kv, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)


def pair(l, r, ls, rs, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def gated(heads, kv, dim, vdim, scale, temp, mlp, kv_from=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


CONFIGS = {
    # small windows that pass over prompts and decoded tokens, part of each head rotated, a layer without feed-forward,
    # a layer that reads another's keys and values, sizes that are multiples of nothing
    "mix": dict(cfg=dict(architecture="Norelix", vocab=300, width=48, norm={"eps": 1e-5}, layers=[
        pair(left(4, 2, 10, 12, 0.3, 12, 3, 4, 100.0), right(2, 1, 9, 10, 3), 0.7, 1.2, dense(40, 1.0)),
        gated(4, 2, 12, 7, 0.25, (0.5, 7), None),
        pair(left(2, 2, 6, 5, 0.4, 5, 0, 6, 10.0), right(3, 3, 5, 7, 2), 1.0, 0.5, dense(24, 3.0)),
        gated(4, 2, 12, 7, 0.3, (0.2, 1), dense(32, 0.5), kv_from=1)]), seed=21, std=0.15, page_size=8),
    # sizes that the tensor-core kernels take; attention first, its keys read again two layers later
    "fast": dict(cfg=dict(architecture="Norelix", vocab=200, width=64, norm={"eps": 3e-6}, layers=[
        gated(4, 1, 16, 24, 0.25, None, dense(48, 2.5)),
        pair(left(2, 2, 32, 16, 0.18, 40, 9, 16, 1e4), right(4, 2, 16, 16, 4), 1.1, 0.9, dense(64, 1.5)),
        gated(4, 1, 16, 24, 0.2, (0.3, 16), dense(48, 2.0), kv_from=0),
        pair(left(8, 1, 8, 8, 0.35, 130, 70, 8, 7.0), right(2, 2, 32, 8, 2), 0.5, 1.0, None)]),
        seed=22, std=0.12, page_size=16),
    # one pair only: one head, a window of one key beside two kept ones, no convolution, no feed-forward
    "lone": dict(cfg=dict(architecture="Norelix", vocab=64, width=20, norm={"eps": 1e-4}, layers=[
        pair(left(1, 1, 4, 3, 0.5, 1, 2, 2, 3.0), right(1, 1, 3, 4, 1), 1.0, 1.0, None),
        pair(left(3, 1, 4, 6, 0.5, 1000, 0, 4, 50.0), right(2, 1, 6, 3, 5), 0.9, 1.4, dense(16, 0.7))]),
        seed=23, std=0.25, page_size=4),
}


@pytest.fixture(scope="module")
def norelix_dirs(tmp_path_factory):
    """Model folders with random weights.  The decays' logarithms are lowered, so that the recurrent state remembers
    for hundreds of tokens and a lost or mixed-up state shows; biases are made as large as the weights' products."""
    from swifttransformer_b200.config import NorelixConfig, save_config
    from swifttransformer_b200.models import build_model_def
    from swifttransformer_b200.weights.random_init import random_tensors
    from swifttransformer_b200.weights.safetensors_io import write_safetensors
    root = tmp_path_factory.mktemp("norelix")
    out = {}
    for name, c in CONFIGS.items():
        cfg = NorelixConfig.from_dict(c["cfg"])
        path = str(root / name)
        save_config(cfg, path)
        tensors = []
        for s, t in random_tensors(build_model_def(cfg).param_specs(), c["seed"], c["std"], "cpu"):
            if s.name.endswith(".A_log"):
                t = (t.float() - 4.0).to(torch.bfloat16)
            elif s.name.endswith(".b") and t.dim() == 1:
                t = (t.float() * 3).to(torch.bfloat16)
            tensors.append((s.name, t))
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
    tol = {"float32": 3e-5, "bfloat16": 5e-2}[dtype]
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        assert got[rid].shape == ref.shape, (what, rid)
        scale = np.abs(ref).max()
        bad = helpers.first_bad(got[rid], ref, tol * scale)
        assert bad is None, (f"{what}/{dtype}: request {rid} first differs at position {bad[0]} of {len(toks)} by "
                             f"{bad[1]:.3e} of {scale:.3e}")
        if dtype == "bfloat16":
            assert np.abs(got[rid] - ref).mean() < 8e-3 * scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("schedule", ["whole", "decode", "portions", "mixed"])
def test_replay_matches_plain(norelix_dirs, name, dtype, schedule):
    from swifttransformer_b200.engine.replay import TraceSession
    reqs = requests_for(name)
    steps = {"whole": helpers.trace_whole, "decode": lambda r: helpers.trace_decode_tail(r, tail=60),
             "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, seed=1, max_live=3)}[schedule](reqs)
    need = helpers.live_token_need(steps)
    s = TraceSession(norelix_dirs[name], dtype, need, page_size=CONFIGS[name]["page_size"], max_requests=3)
    got = helpers.replay(s, steps)
    compare(norelix_dirs[name], reqs, got, dtype, f"{name}/{schedule}")
    s.cache.check()
    assert all(g.pool.num_held == 0 for g in s.cache.groups)


def test_residual_stream_after_every_layer(norelix_dirs):
    """Layer by layer: the float residual rows after every layer (what is still pending included)."""
    from swifttransformer_b200.engine.replay import TraceSession
    for name in CONFIGS:
        toks = helpers.random_tokens(CONFIGS[name]["cfg"]["vocab"], 29, seed=5)
        s = TraceSession(norelix_dirs[name], "float32", 64, page_size=CONFIGS[name]["page_size"], max_requests=1)
        s.runner.use_cuda_graphs = False
        got = []

        def hook(i, stream):
            x, p = stream.x.clone(), stream.pending
            for part in ((p.value,) if p and p.value is not None else ()) + ((p.parts.sum(0),) if p and p.parts is not None else ()):
                x += part.float()
            if p and p.bias is not None:
                x += p.bias
            got.append(x.cpu().numpy())
        s.model.after_layer = hook
        s.run_step([dict(id="a", tokens=toks, want=[28])], ["a"])
        cfg, w = pn.load_model(norelix_dirs[name])
        _, ref = pn.forward(cfg, w, toks, return_layers=True)
        assert len(got) == len(ref) == len(cfg["layers"])
        for i in range(len(ref)):
            assert np.abs(got[i] - ref[i]).max() < 2e-5 * np.abs(ref[i]).max(), (name, i)


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_and_eager_steps_agree(norelix_dirs, dtype):
    from swifttransformer_b200.engine.replay import TraceSession
    reqs = requests_for("fast", lengths=(70, 9))
    steps = helpers.trace_mixed(reqs, seed=2, max_live=2)
    outs = []
    for graphs in (True, False):
        s = TraceSession(norelix_dirs["fast"], dtype, helpers.live_token_need(steps), max_requests=2)
        s.runner.use_cuda_graphs = graphs
        outs.append(helpers.replay(s, steps))
        assert (s.runner.graph_steps + s.runner.padded_graph_steps > 0) == graphs
    for rid in reqs:
        tol = 1e-5 if dtype == "float32" else 3e-2
        err = np.abs(outs[0][rid] - outs[1][rid]).max(axis=1) / np.abs(outs[1][rid]).max()
        assert err.max() < tol, (rid, int(np.argmax(err)), float(err.max()))


@pytest.mark.parametrize("name", ["mix", "fast"])
def test_long_decoding_with_pages_and_slots_used_again(norelix_dirs, name):
    """Three requests after one another through the same single slot and a pool that holds only one of them, each
    decoded token by token for 300 steps after a short prompt: the windows pass over decoded tokens, their pages come
    back, and the next request starts from a zero state in the slot the last one left."""
    from swifttransformer_b200.engine.replay import TraceSession
    ps = CONFIGS[name]["page_size"]
    s = TraceSession(norelix_dirs[name], "float32", 384, page_size=ps, max_requests=1)
    for k in range(3):
        toks = helpers.random_tokens(CONFIGS[name]["cfg"]["vocab"], 330, seed=40 + k)
        rows = [s.run_step([dict(id=k, tokens=toks[:30], want=list(range(30)))]).cpu().numpy().copy()]
        for t in range(30, 330):
            rows.append(s.run_step([dict(id=k, tokens=[toks[t]], want=[0])], [k] if t == 329 else []).cpu().numpy().copy())
        s.check()
        ref = plain_logits(norelix_dirs[name], toks)
        bad = helpers.first_bad(np.concatenate(rows), ref, 3e-5 * np.abs(ref).max())
        assert bad is None, (k, bad)
    assert all(g.pool.num_held == 0 for g in s.cache.groups)


def test_a_window_gives_its_pages_back(norelix_dirs):
    """A model whose every attention has a window holds, however long the request grows, only the pages of the window
    and of the kept first keys."""
    from swifttransformer_b200.engine.replay import TraceSession
    s = TraceSession(norelix_dirs["lone"], "float32", 2048, page_size=4, max_requests=1)
    toks = helpers.random_tokens(64, 600, seed=9)
    s.run_step([dict(id=0, tokens=toks[:500], want=[])])
    held = [g.pool.num_held for g in s.cache.groups]
    got = s.run_step([dict(id=0, tokens=toks[500:], want=[99])]).cpu().numpy()
    # the second layer's window (1000 keys) is longer than the request: its group holds every page; the first layer's
    # group holds the kept first page and the window's
    assert sorted(held)[0] <= 3 and sorted(held)[-1] >= 500 // 4, held
    ref = plain_logits(norelix_dirs["lone"], toks)
    assert np.abs(got[0] - ref[599]).max() < 3e-5 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "fast"])
def test_greedy_generation_through_the_engine(norelix_dirs, name, dtype):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.sampling.sampler import SamplingParams
    vocab = CONFIGS[name]["cfg"]["vocab"]
    prompts = [helpers.random_tokens(vocab, n, seed=n) for n in (5, 31, 1, 18, 44, 9)]
    eng = LLMEngine(norelix_dirs[name], dtype=dtype, page_size=CONFIGS[name]["page_size"], num_pages=24,
                    max_num_seqs=3, max_batch_tokens=48, chunk_size=20, max_seq_len=256)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0))
    cfg, w = pn.load_model(norelix_dirs[name])
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


def test_run_gpt_takes_a_norelix_folder(norelix_dirs, tmp_path):
    import subprocess
    import sys
    vocab = CONFIGS["mix"]["cfg"]["vocab"]
    prompts = [helpers.random_tokens(vocab, n, 70 + n) for n in (6, 21)]
    inp = tmp_path / "in.txt"
    inp.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_gpt"), norelix_dirs["mix"], "any", "fp32", str(inp),
                        "--max_decoding_step", "5", "--num_total_blocks", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = pn.load_model(norelix_dirs["mix"])
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 2
    for line, p in zip(lines, prompts):
        got = [int(t) for t in line.split(")")[1].split("(")[0].split()]
        assert got == pn.greedy(cfg, w, p, 5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program_with_four_slots(norelix_dirs, tmp_path, dtype):
    """bin/trace_run with its defaults (four request slots, pages of 16): six requests, at most four live, so slots and
    pages are handed out again; every wanted row against the plain implementation."""
    import subprocess
    import sys
    name = "fast"
    reqs = requests_for(name, lengths=(50, 1, 33, 170, 18, 40))
    steps = helpers.trace_mixed(reqs, seed=3, max_live=4)
    out = tmp_path / "out"
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", norelix_dirs[name], "--dtype", dtype,
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
    compare(norelix_dirs[name], reqs, {rid: np.concatenate(v) for rid, v in got.items()}, dtype, "trace_run")
