"""A plain, slow implementation of the Nafelix design in numpy float64, one function per mechanism.

It shares no code with the package: it has its own safetensors reader, reads ``config.json`` as a dict and walks
whole sequences without any cache.  Notation: T tokens, W the model width, H query (or value) heads, G key/value
(or query/key) heads, d the key size, e the value size; a head a reads group a // (H / G).

  streams      n copies x_1..x_n of the residual rows; a sub-layer reads u = sum_s a_s x_s and its result y goes back
               as x_t <- sum_s M[s, t] x_s + b_t y; the model's residual is the sum of the copies
  sub-layer    y = f(c(N(u))) with N an RMS norm with a weight and c(h) = h + causal convolution of h over time
  talking      windowed attention with a learned extra logit per head in the softmax's denominator whose weights are
               mixed over heads (P'_a = sum_b T[a, b] P_b) before they meet the values of head a's own group
  gated delta  S <- g S;  r = beta (v - S^T k);  S <- S + k r^T;  o = S^T q      per value head, g one number per token
  experts      the ``top`` largest of softmax(router logits), renormalised, over clamped gated units
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, shape = data[lo:hi], info["shape"]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: unexpected dtype {info['dtype']}")
        out[name] = a.reshape(shape)
    return out


def load_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ------------------------------------------------------------------ elementary functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(y, eps):
    """y divided by its root mean square over the last axis, eps inside the root."""
    return y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + eps)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    neg = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, aq * (np.expm1(neg) - neg) + 0.5 * z)


def causal_conv(h, f):
    """out_t = sum_j f[:, j] h_(t - taps + 1 + j), zeros before the start.  h [T, C], f [C, taps]."""
    T, taps = h.shape[0], f.shape[1]
    out = np.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += f[:, j] * h[:T - back]
    return out


def rotate_halves(u, positions, dims, base):
    """u [T, heads, d]: dimension i < dims/2 is paired with i + dims/2; the pair turns by p * base^(-2i/dims)."""
    if not dims:
        return u
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = u.copy()
    a, b = u[..., :half], u[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def seen_window(T, size):
    """[T, T]: query i sees key j when 0 <= i - j < size (size None: every earlier key and itself)."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (i - j >= 0) & ((i - j < size) if size else True)


def window_of(mx):
    return mx["mask"]["size"] if mx.get("mask") else None


def rotated(u, positions, mx):
    rot = mx.get("rot")
    return rotate_halves(u, positions, rot["dims"], rot["base"]) if rot else u


def softmax_with_sink(s, seen, sink):
    """Rows of s [H, T, T] over the seen keys; the denominator also holds exp(sink[a]) for head a."""
    s = np.where(seen[None], s, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink[:, None, None])
    p = np.exp(s - m)
    return p / (p.sum(axis=-1, keepdims=True) + np.exp(sink[:, None, None] - m))


def attention_weights(q, k, seen, scale, sink):
    """q [T, H, d], k [T, G, d] -> softmax weights [H, T, T]."""
    H, G = q.shape[1], k.shape[1]
    grp = np.arange(H) // (H // G)
    s = np.einsum("iad,jad->aij", q, k[:, grp, :]) * scale
    return softmax_with_sink(s, seen, sink)


def apply_weights(P, v):
    """P [H, T, T], v [T, G, e] -> [T, H, e]; head a reads the values of its own group."""
    H, G = P.shape[0], v.shape[1]
    grp = np.arange(H) // (H // G)
    return np.einsum("aij,jae->iae", P, v[:, grp, :])


# ------------------------------------------------------------------ mixers
def talking_attention(h, w, p, mx):
    """The left member of a pair: no biases, rotation on part of each head, window, sink, mixed heads, a gate
    number per head."""
    T = h.shape[0]
    H, G, d, e = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, e)
    q, k = rotated(q, pos, mx), rotated(k, pos, mx)
    P = attention_weights(q, k, seen_window(T, window_of(mx)), mx["scale"], w[p + "sink"])
    P = np.einsum("ab,bij->aij", w[p + "talk"], P)
    o = apply_weights(P, v)
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * e) @ w[p + "o"].T


def gated_attention(h, w, p, mx, eps):
    """The 'attention' mixer: biased projections, rotation, q and k divided by their root mean square, window,
    sink, an element-wise sigmoid gate."""
    T = h.shape[0]
    H, G, d, e = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, e)
    q, k = rms_unit(rotated(q, pos, mx), eps), rms_unit(rotated(k, pos, mx), eps)
    P = attention_weights(q, k, seen_window(T, window_of(mx)), mx["scale"], w[p + "sink"])
    o = apply_weights(P, v).reshape(T, H * e)
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def delta_rule(q, k, v, g, beta):
    """q, k [T, H, d], v [T, H, e], g and beta [T, H] -> o [T, H, e]; the state starts at zero."""
    T, H, d = q.shape
    e = v.shape[2]
    S = np.zeros((H, d, e))
    o = np.zeros((T, H, e))
    for t in range(T):
        S = S * g[t][:, None, None]
        r = beta[t][:, None] * (v[t] - np.einsum("ade,ad->ae", S, k[t]))
        S = S + k[t][:, :, None] * r[:, None, :]
        o[t] = np.einsum("ade,ad->ae", S, q[t])
    return o


def gated_delta(h, w, p, mx, eps):
    """The right member of a pair."""
    T = h.shape[0]
    H, G, d, e = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]

    def branch(name):
        return silu(causal_conv(h @ w[p + name].T, w[p + name + ".conv"]))

    q, k, v = branch("q").reshape(T, G, d), branch("k").reshape(T, G, d), branch("v").reshape(T, H, e)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    grp = np.arange(H) // (H // G)
    beta = sigmoid(h @ w[p + "b"].T)
    g = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_rule(q[:, grp, :], k[:, grp, :], v, g, beta)
    o = rms_unit(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).reshape(T, H, e)
    return o.reshape(T, H * e) @ w[p + "o"].T


def parallel_mixer(h, w, p, mx, eps):
    a = rms_unit(talking_attention(h, w, p + "left.", mx["left"]), eps) * w[p + "left.out"]
    b = rms_unit(gated_delta(h, w, p + "right.", mx["right"], eps), eps) * w[p + "right.out"]
    return 0.5 * (a + b)


# ------------------------------------------------------------------ feed-forward
def dense_ff(h, w, p):
    pq = w[p + "act"]
    return xielu(h @ w[p + "up"].T, pq[0], pq[1]) @ w[p + "down"].T


def clamped_unit(a, b, limit):
    g, u = np.minimum(a, limit), np.clip(b, -limit, limit)
    return g * sigmoid(1.702 * g) * (u + 1.0)


def route(h, w_router, top):
    """-> (chosen [T, top], weights [T, top]): the largest scores of softmax(z), divided by their sum."""
    z = h @ w_router.T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    sc = np.take_along_axis(s, chosen, axis=-1)
    return chosen, sc / (sc.sum(-1, keepdims=True) + 1e-20)


def experts_ff(h, w, p, mlp):
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    chosen, weights = route(h, w[p + "router"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for c, wt in zip(chosen[t], weights[t]):
            e = f"{p}e{c}."
            out[t] += wt * (clamped_unit(h[t] @ w[e + "gate"].T, h[t] @ w[e + "up"].T, limit) @ w[e + "down"].T)
    return out


def feed_forward(h, w, p, mlp):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else experts_ff(h, w, p, mlp)


# ------------------------------------------------------------------ the model
def layer_runs(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer_input(xs, w, hc, norm, canon, eps):
    u = np.einsum("s,stw->tw", w[hc + ".in"], xs)
    h = rms_unit(u, eps) * w[norm]
    return h + causal_conv(h, w[canon]) if canon in w else h


def streams_update(xs, y, w, hc):
    return np.einsum("st,siw->tiw", w[hc + ".mix"], xs) + w[hc + ".out"][:, None, None] * y[None]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the summed residual rows after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    xs = np.repeat(x[None], cfg.get("streams") or 1, axis=0)
    after = []
    for i in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        h = sublayer_input(xs, w, p + "hc1", p + "norm1", p + "canon1", eps)
        if layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            y = gated_attention(h, w, p + "mix.", layer["mixer"], eps)
        xs = streams_update(xs, y, w, p + "hc1")
        if layer.get("mlp") is not None:
            h = sublayer_input(xs, w, p + "hc2", p + "norm2", p + "canon2", eps)
            xs = streams_update(xs, feed_forward(h, w, p + "mlp.", layer["mlp"]), w, p + "hc2")
        after.append(xs.sum(0))
    x = rms_unit(xs.sum(0), eps) * w["final.norm"]
    logits = x @ w["head"].T
    return (logits, np.stack(after)) if return_layers else logits


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
