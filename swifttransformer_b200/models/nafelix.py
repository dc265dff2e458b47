"""Nafelix put together from the parts.

A decoder-only model with ``streams`` copies of the residual rows whose layers are listed in the configuration:

  embedding     x = embed[token]; every copy starts as x
  layer i       for the mixer and then the feed-forward (which may be absent), with the layer's coefficients
                'l<i>.hc1.*' / 'l<i>.hc2.*':  u = sum_s in[s] x_s;  h = N(u);  h <- h + conv(h) ('l<i>.canon1/2');
                y = sub-layer(h);  x_t <- sum_s mix[s, t] x_s + out[t] y            (block ``hyper_pre_norm``)
  'parallel'    (N_l(left(h)) + N_r(right(h))) / 2, each result RMS-normed over the width with a weight of its own
                                                                                     (``side_by_side`` with norms)
                left:  grouped attention without biases, halves rotation on part of each head, a window, a learned
                       extra logit per head in the softmax's denominator, the heads' weights mixed by a matrix, one
                       sigmoid gate number per head         (``grouped_attention`` with talk_name, gate="head")
                right: the gated delta rule with one decay per head and a full SiLU output gate
                                                            (``gated_delta_rule`` with low_rank=False)
  'attention'   grouped attention with biased q, k, v, rotation, q and k divided by their root mean square, a window,
                a learned extra logit per head, an element-wise sigmoid gate        (``grouped_attention``)
  feed-forward  'dense': down(act(up h)) with the two-sided activation of two learned numbers  (``dense_xielu``)
                'moe':   softmax router, the ``top`` largest renormalised, clamped gated experts
                                                                                     (``routed_experts`` with limit)
  loop          layers start..stop-1 run ``times`` times in a row with the same weights; every run has cache
                entries of its own
  output        N(sum of the copies) with 'final.norm', then the product with 'head'

Tensor names are those of the design's checkpoints.  The model has no position table and no context limit of its own.
"""
from __future__ import annotations

from ..config.nafelix import NafelixConfig
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from ..parts.embedding import Embedding, OutputHead
from .base import LayerStep, ModelDef
from .registry import register_model

# constants of the design's expert unit: g * sigmoid(GATE_ALPHA * g) * (u + UP_SHIFT)
GATE_ALPHA = 1.702
UP_SHIFT = 1.0
# the dense feed-forward's activation on the negative side has the factor XIELU_SHIFT + softplus(q)
XIELU_SHIFT = 0.5
# a pair's result is the mean of its two normed members
PAIR_WEIGHTS = (0.5, 0.5)


def _rotation(mx):
    rot = mx.get("rot")
    return POSITION_ENCODINGS.build("rotary_halves", dims=rot["dims"], base=rot["base"]) if rot and rot["dims"] else None


def _window(mx):
    return mx["mask"]["size"] if mx.get("mask") else None


def _left(W, m, mx):
    return MIXERS.build(
        "grouped_attention", hidden=W, num_heads=mx["heads"], num_kv_heads=mx["kv_heads"], dim=mx["dim"],
        vdim=mx["vdim"], scale=mx["scale"], names={k: m + k for k in ("q", "k", "v", "o", "g")}, qkv_bias=False,
        o_bias=False, window=_window(mx), qk_position=_rotation(mx), sink_name=m + "sink", talk_name=m + "talk",
        gate="head", float_out=True)


def _right(W, m, mx, eps):
    keys = ("q", "k", "v", "b", "a", "g", "o", "A_log", "dt_bias", "norm")
    return MIXERS.build("gated_delta_rule", hidden=W, num_heads=mx["heads"], num_qk_heads=mx["kv_heads"], dim=mx["dim"],
                        vdim=mx["vdim"], conv_taps=mx["conv"], eps=eps, names={k: m + k for k in keys},
                        float_out=True, low_rank=False, gate_act="silu")


def _feed_forward(W, p, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return FEED_FORWARDS.build("dense_xielu", hidden=W, inner=mlp["ff"], up_name=p + "up", down_name=p + "down",
                                   act_name=p + "act", shift=XIELU_SHIFT, float_out=True)
    n = mlp["router"]["experts"]
    names = [{k: f"{p}e{e}.{k}" for k in ("gate", "up", "down")} for e in range(n)]
    return FEED_FORWARDS.build("routed_experts", hidden=W, inner=mlp["expert"]["ff"], num_experts=n,
                               top=mlp["router"]["top"], activation="none", expert_names=names,
                               router_name=p + "router", renormalise=True, limit=mlp["expert"]["limit"],
                               alpha=GATE_ALPHA, shift=UP_SHIFT)


@register_model(NafelixConfig.ARCHITECTURE)
def build_nafelix(cfg: NafelixConfig) -> ModelDef:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding(cfg.vocab, W, W, "embed")
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer["mixer"]
        m = p + "mix."
        if layer["type"] == "parallel":
            mixer = MIXERS.build("side_by_side", left=_left(W, m + "left.", mx["left"]),
                                 right=_right(W, m + "right.", mx["right"], eps),
                                 norm_names=(m + "left.out", m + "right.out"), width=W, eps=eps, weights=PAIR_WEIGHTS)
        else:
            mixer = MIXERS.build(
                "grouped_attention", hidden=W, num_heads=mx["heads"], num_kv_heads=mx["kv_heads"], dim=mx["dim"],
                vdim=mx["vdim"], scale=mx["scale"], names={k: m + k for k in ("q", "k", "v", "o", "g")}, qkv_bias=True,
                o_bias=False, window=_window(mx), qk_position=_rotation(mx), sink_name=m + "sink", gate=True,
                qk_norm_eps=eps, float_out=True)
        ffn = _feed_forward(W, p + "mlp.", layer.get("mlp"))
        norm = lambda name: NORMS.build("rmsnorm", width=W, eps=eps, name=name)
        blocks.append(BLOCKS.build(
            "hyper_pre_norm", mixer=mixer, feed_forward=ffn, norm1=norm(p + "norm1"),
            norm2=norm(p + "norm2") if ffn is not None else None, streams=cfg.streams, width=W,
            hc_names=(p + "hc1", p + "hc2"), canon_names=(p + "canon1", p + "canon2") if cfg.canon_taps else None,
            taps=cfg.canon_taps or 1))
    # every run of a layer (a looped layer runs several times) has a cache entry of its own
    order = [LayerStep(block=i, cache=run) for run, i in enumerate(cfg.layer_runs())]
    final_norm = NORMS.build("rmsnorm", width=W, eps=eps, name="final.norm")
    head = OutputHead(cfg.vocab, W, W, "head")
    return ModelDef(cfg, embedding, POSITION_ENCODINGS.build("none"), blocks, order, final_norm, head)
