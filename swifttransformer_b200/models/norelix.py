"""Norelix put together from the parts.

A decoder-only model whose layers are listed in the configuration:

  embedding     x = embed[token]
  layer i       x <- x + mixer(N1(x));  x <- x + ff(N2(x))                         (block ``pre_norm``; the
                feed-forward and N2 may be absent)      N: RMS norm with a weight vector ('l<i>.norm1', 'l<i>.norm2')
  'parallel'    a * left(h) + b * right(h), both reading the same h                 (``side_by_side``)
                left:  grouped attention with biased q, k, v, halves rotation on part of each head, a window of
                       recent keys plus the request's first keys, and one added to the softmax's denominator
                       (``grouped_attention`` with window, keep_first, sink = 0)
                right: the gated delta rule                                          (``gated_delta_rule``)
  'attention'   grouped attention with biased q, k, v and output, a query temperature that grows with the
                logarithm of the position, all earlier keys, a sigmoid gate on the heads' results; with
                ``kv_from`` it has no key and value projections and reads another layer's pages
                (``grouped_attention`` with q_temp, gate, own_kv; the layer step points at the other entry)
  feed-forward  down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate h, limit), u = clamp(up h, +-limit), all
                biased                                                              (``gated_clamped``)
  output        N(x) with 'final.norm', then the product with 'head'

Tensor names are those of the design's checkpoints: 'embed', 'l<i>.norm1/2', 'l<i>.mix.*' ('left.*' and 'right.*'
in a parallel layer), 'l<i>.mlp.*', 'final.norm', 'head'.  The model has no position table and no context limit of
its own.
"""
from __future__ import annotations

from ..config.norelix import NorelixConfig
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from ..parts.embedding import Embedding, OutputHead
from .base import LayerStep, ModelDef
from .registry import register_model

# constants of the design's feed-forward unit: g * sigmoid(GATE_ALPHA * g) * (u + UP_SHIFT)
GATE_ALPHA = 1.702
UP_SHIFT = 1.0
# the logit of the term that the left attention's softmax adds to its denominator (exp(0) = 1)
LEFT_SINK = 0.0


def _left(W, m, mx, out_scale):
    rot, mask = mx.get("rot"), mx.get("mask")
    return MIXERS.build(
        "grouped_attention", hidden=W, num_heads=mx["heads"], num_kv_heads=mx["kv_heads"], dim=mx["dim"],
        vdim=mx["vdim"], scale=mx["scale"], names={k: m + k for k in ("q", "k", "v", "o")}, qkv_bias=True, o_bias=False,
        window=mask["size"] if mask else None, keep_first=(mask.get("keep_first") or 0) if mask else 0, sink=LEFT_SINK,
        qk_position=POSITION_ENCODINGS.build("rotary_halves", dims=rot["dims"], base=rot["base"])
        if rot and rot["dims"] else None, out_scale=out_scale)


def _right(W, m, mx, eps, out_scale):
    keys = ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o", "A_log", "dt_bias", "norm")
    return MIXERS.build("gated_delta_rule", hidden=W, num_heads=mx["heads"], num_qk_heads=mx["kv_heads"], dim=mx["dim"],
                        vdim=mx["vdim"], conv_taps=mx["conv"], eps=eps, names={k: m + k for k in keys},
                        out_scale=out_scale, float_out=True, rank=mx.get("rank", 16))


@register_model(NorelixConfig.ARCHITECTURE)
def build_norelix(cfg: NorelixConfig) -> ModelDef:
    W, eps = cfg.width, cfg.norm_eps
    embedding = Embedding(cfg.vocab, W, W, "embed")
    blocks, order, entry_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer["mixer"]
        m = p + "mix."
        if layer["type"] == "parallel":
            ls = mx["left_scale"] if mx.get("left_scale") is not None else 1.0
            rs = mx["right_scale"] if mx.get("right_scale") is not None else 1.0
            mixer = MIXERS.build("side_by_side", left=_left(W, m + "left.", mx["left"], ls),
                                 right=_right(W, m + "right.", mx["right"], eps, rs))
        else:
            own = mx.get("kv_from") is None
            qt = mx.get("q_temp")
            mixer = MIXERS.build(
                "grouped_attention", hidden=W, num_heads=mx["heads"], num_kv_heads=mx["kv_heads"], dim=mx["dim"],
                vdim=mx["vdim"], scale=mx["scale"], names={k: m + k for k in ("q", "k", "v", "o", "g")}, qkv_bias=True,
                o_bias=True, q_temp=(qt["coef"], qt["every"]) if qt else None, gate=True, own_kv=own)
        mlp = layer.get("mlp")
        ffn = FEED_FORWARDS.build("gated_clamped", hidden=W, inner=mlp["ff"], limit=mlp["limit"], alpha=GATE_ALPHA,
                                  shift=UP_SHIFT, gate_name=p + "mlp.gate", up_name=p + "mlp.up",
                                  down_name=p + "mlp.down") if mlp is not None else None
        norm = lambda name: NORMS.build("rmsnorm", width=W, eps=eps, name=name)
        blocks.append(BLOCKS.build("pre_norm", mixer=mixer, feed_forward=ffn, norm1=norm(p + "norm1"),
                                   norm2=norm(p + "norm2") if ffn is not None else None))
        src = cfg.kv_source(i) if layer["type"] == "attention" else i
        if src == i:
            entry_of[i] = len(entry_of)
        order.append(LayerStep(block=i, cache=entry_of[src], writes_cache=src == i))
    final_norm = NORMS.build("rmsnorm", width=W, eps=eps, name="final.norm")
    head = OutputHead(cfg.vocab, W, W, "head")
    return ModelDef(cfg, embedding, POSITION_ENCODINGS.build("none"), blocks, order, final_norm, head)
