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
