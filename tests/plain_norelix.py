"""A plain, slow Norelix: whole sequences, no cache, one function per mechanism.

This file is the tests' oracle for the Norelix design.  It shares no code with
the package: it reads config.json and the safetensors file itself and computes
with numpy in float64.  The notation, for a sequence of T tokens at positions
0..T-1 (x: the residual stream [T, width]):

  layer            x <- x + mixer(N1(x));  x <- x + ff(N2(x))        (the feed-forward may be absent)
  N(y)             y / sqrt(mean(y^2) + eps) * w
  mixer 'attention'  grouped heads, biased projections, queries scaled by a temperature that grows with the
                   logarithm of the position, causal softmax, a sigmoid gate on the concatenated heads, biased
                   output projection; a layer may read another layer's keys and values
  mixer 'parallel' a * left + b * right, both reading the same input:
                   left   grouped heads, biased projections, part of each head rotated by position (halves),
                          a window of recent keys plus the first few keys of the sequence, one added to the
                          softmax's denominator
                   right  the gated delta rule: short convolutions with silu on q, k, v, unit q and k, a
                          decay per head and key channel, a write strength per head, a state matrix per head
                          updated token by token, a normed and gated read-out
  feed-forward     g = min(gate h, L), u = clamp(up h, -L, L), down(g sigmoid(1.702 g) (u + 1)), all biased
  output           N(x) with the final weight, product with the head matrix
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_safetensors(path):
    """name -> float64 (or integer) array."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        b, e = rec["data_offsets"]
        raw = data[b:e]
        if rec["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        elif rec["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype=np.float32).astype(np.float64)
        elif rec["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype=np.int32)
        else:
            raise ValueError(f"unexpected tensor type {rec['dtype']}")
        out[name] = arr.reshape(rec["shape"])
    return out


def load_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------

def rms(y, eps):
    """y / sqrt(mean(y^2) + eps) over the last axis."""
    return y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rotate_halves(u, positions, dims, base):
    """u [T, heads, n]: of the first `dims` dimensions, i is paired with i + dims/2 and the pair turned by
    p * base^(-2i/dims); the other dimensions pass unchanged."""
    out = u.copy()
    half = dims // 2
    p = np.asarray(positions, dtype=np.float64)[:, None]
    for i in range(half):
        a = p * base ** (-2.0 * i / dims)
        c, s = np.cos(a), np.sin(a)
        lo, hi = u[..., i], u[..., i + half]
        out[..., i] = lo * c - hi * s
        out[..., i + half] = hi * c + lo * s
    return out


def seen_window(T, size, keep_first):
    """[T, T] bool: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def seen_causal(T):
    return np.arange(T)[None, :] <= np.arange(T)[:, None]


def softmax_rows(s, seen, one_more):
    """Softmax over the seen keys of every row; `one_more`: a term exp(0) joins the denominator (and nothing
    else)."""
    s = np.where(seen, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if one_more:
        m = np.maximum(m, 0.0)
    e = np.exp(s - m)
    den = e.sum(axis=-1, keepdims=True)
    if one_more:
        den = den + np.exp(-m)
    return e / den


def temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = np.asarray(positions)
    return 1.0 + coef * np.log(np.floor((p + 1) / every) + 1.0)


def grouped_attention(q, k, v, seen, scale, one_more):
    """q [T, H, d], k [T, G, d], v [T, G, vd] -> [T, H * vd]; head a reads key/value head a // (H / G)."""
    T, H, _ = q.shape
    G, vd = k.shape[1], v.shape[2]
    out = np.zeros((T, H, vd))
    for a in range(H):
        g = a // (H // G)
        p = softmax_rows(q[:, a] @ k[:, g].T * scale, seen, one_more)
        out[:, a] = p @ v[:, g]
    return out.reshape(T, H * vd)


def windowed_attention(h, w, p, mx):
    """The left half of a 'parallel' mixer.  h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, G, d, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, vd)
    rot = mx.get("rot")
    if rot and rot["dims"]:
        q, k = rotate_halves(q, pos, rot["dims"], rot["base"]), rotate_halves(k, pos, rot["dims"], rot["base"])
    seen = seen_window(T, mx["mask"]["size"], mx["mask"]["keep_first"])
    o = grouped_attention(q, k, v, seen, mx["scale"], one_more=True)
    return o @ w[p + "o"].T


def causal_conv(u, f):
    """u [T, C], f [C, taps] -> out[t, c] = sum_j f[c, j] * u[t - taps + 1 + j, c], zeros before the start."""
    T, taps = u.shape[0], f.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], axis=0)
    out = np.zeros_like(u)
    for j in range(taps):
        out += padded[j:j + T] * f[:, j]
    return out


def unit(y):
    return y / np.sqrt(np.sum(y * y, axis=-1, keepdims=True) + 1e-6)


def delta_rule(q, k, v, decay, beta):
    """One head.  q, k, decay [T, d], v [T, vd], beta [T] -> o [T, vd].  The state S [d, vd] starts at zero:
    S <- decay_t (rows) * S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]))
    o = np.zeros_like(v)
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def gated_delta(h, w, p, mx, eps):
    """The right half of a 'parallel' mixer.  h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, G, d, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = unit(silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)) * d ** -0.5
    k = unit(silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d))
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, vd)
    beta = sigmoid(h @ w[p + "b"].T)                                             # [T, H]
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, d)
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * step)                # [T, H, d]
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, vd)
    out = np.zeros((T, H, vd))
    for a in range(H):
        g = a // (H // G)
        o = delta_rule(q[:, g], k[:, g], v[:, a], decay[:, a], beta[:, a])
        out[:, a] = rms(o, eps) * w[p + "norm"] * gate[:, a]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def parallel_mixer(h, w, p, mx, eps):
    return (mx["left_scale"] * windowed_attention(h, w, p + "left.", mx["left"])
            + mx["right_scale"] * gated_delta(h, w, p + "right.", mx["right"], eps))


def keys_values(h, w, p, mx):
    T = h.shape[0]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, mx["kv_heads"], mx["dim"])
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, mx["kv_heads"], mx["vdim"])
    return k, v


def gated_attention(h, w, p, mx, kv):
    """The 'attention' mixer; kv: the keys and values it reads (its own, or another layer's)."""
    T = h.shape[0]
    H, d = mx["heads"], mx["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    qt = mx.get("q_temp")
    if qt:
        q = q * temperature(np.arange(T), qt["coef"], qt["every"])[:, None, None]
    o = grouped_attention(q, kv[0], kv[1], seen_causal(T), mx["scale"], one_more=False)
    o = o * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T + w[p + "o.b"]


def clamped_unit(a, b, limit):
    """g = min(a, limit), u = clamp(b, -limit, limit): g * sigmoid(1.702 g) * (u + 1)."""
    g = np.minimum(a, limit)
    u = np.clip(b, -limit, limit)
    return g * sigmoid(1.702 * g) * (u + 1.0)


def feed_forward(h, w, p, mlp):
    y = clamped_unit(h @ w[p + "gate"].T + w[p + "gate.b"], h @ w[p + "up"].T + w[p + "up.b"], mlp["limit"])
    return y @ w[p + "down"].T + w[p + "down.b"]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)].copy()
    after, kept = [], {}
    for i, spec in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", spec["mixer"]
        h = rms(x, eps) * w[p + "norm1"]
        if spec["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", mx, eps)
        elif spec["type"] == "attention":
            if mx.get("kv_from") is None:
                kept[i] = keys_values(h, w, p + "mix.", mx)
            y = gated_attention(h, w, p + "mix.", mx, kept[mx.get("kv_from", i) if mx.get("kv_from") is not None else i])
        else:
            raise ValueError(f"unknown layer type {spec['type']}")
        x = x + y
        if spec.get("mlp") is not None:
            x = x + feed_forward(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", spec["mlp"])
        after.append(x.copy())
    y = rms(x, eps) * w["final.norm"]
    logits = y @ w["head"].T
    return (logits, np.stack(after)) if return_layers else logits


def greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
