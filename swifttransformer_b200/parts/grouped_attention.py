"""Grouped-query attention with its options as constructor arguments.

Per query head a (key/value head a // (heads / kv_heads)), key/query size ``dim``, value size ``vdim``:

    q, k, v   = the projections of the mixer's input (+ biases)
    q, k      <- rotated by position on the first ``rot.dims`` dimensions (a ``rotary_halves`` encoding), or not
    q         <- q * (1 + coef * ln(floor((p + 1) / every) + 1))            (``q_temp`` = (coef, every), or None)
    s_j       = scale * q . k_j  over the keys the query at p sees: j <= p, and with a ``window``
                p - j < window or j < keep_first
    q, k      <- q / rms(q), k / rms(k) over ``dim``, after the rotation   (``qk_norm_eps``, or None)
    w_j       = exp(s_j) / (sum_i exp(s_i) [+ exp(sink)])                  (``sink``: a logit, or None; ``sink_name``:
                                                                            a learned logit per head)
    w_a(j)    <- sum_b T[a, b] w_b(j)                                      (``talk_name``: T [heads, heads] mixes the
                                                                            heads' normalised weights; the extra
                                                                            term's share is not mixed)
    o         = out_scale * sum_j w_j v_j  [* sigmoid(W_g h)]              (``gate``: a projection of the same input,
                                                                            True: a number per (head, value dimension),
                                                                            "head": one number per head)

and the heads' results go through the output projection.  ``own_kv`` False: the mixer has no key and value
projections and reads the pages another layer step fills (the model's layer order points it at that entry).

The cache holds, per key/value head and position, the key (after bias and rotation) and the value, in pages
(``PagedKVSpec`` with ``value_dim``); under a window the pages behind it are given back, except those that hold
the first ``keep_first`` positions.  One fused product gives q | k | v | gate logits; ``gqa_prepare`` adds the
biases, rotates, scales the queries and writes the pages; the attention kernels apply gate and out_scale when
they store a head's result.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, ParamSpec
from .attention import PagedAttentionPlan
from .base import MIXERS, Delta, Mixer, PagedKVSpec, StepPlan


@MIXERS.register("grouped_attention")
class GroupedAttention(Mixer):
    """names: tensor names of the projections {"q","k","v","o"} and, with ``gate``, "g" ([out, in] matrices);
    a projection's bias is its name + ``bias_suffix``.  ``qkv_bias`` / ``o_bias``: which projections have one."""

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 names: Dict[str, str], qkv_bias: bool = True, o_bias: bool = False, bias_suffix: str = ".b",
                 window: Optional[int] = None, keep_first: int = 0, sink: Optional[float] = None,
                 qk_position: Any = None, q_temp: Optional[Tuple[float, int]] = None, gate: Any = False,
                 out_scale: float = 1.0, own_kv: bool = True, sink_name: Optional[str] = None,
                 talk_name: Optional[str] = None, qk_norm_eps: Optional[float] = None, float_out: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads")
        if window is not None and window <= 0:
            raise ValueError("a window holds at least one key")
        if keep_first < 0 or (keep_first and window is None):
            raise ValueError("'keep_first' needs a window and must not be negative")
        if q_temp is not None and int(q_temp[1]) <= 0:
            raise ValueError("the query temperature's period must be positive")
        if gate not in (False, True, None, "head"):
            raise ValueError("'gate' is False, True (a number per head and value dimension) or 'head'")
        if sink is not None and sink_name:
            raise ValueError("the softmax's extra term is one constant logit or a learned one per head, not both")
        self.hidden, self.nh, self.nkv, self.dim, self.vdim = hidden, num_heads, num_kv_heads, dim, vdim
        self.scale, self.names, self.suffix = float(scale), dict(names), bias_suffix
        self.qkv_bias, self.o_bias = qkv_bias, o_bias
        self.window, self.keep_first = (int(window) if window else None), int(keep_first)
        self.sink = None if sink is None else float(sink)
        self.qk_position = qk_position
        self.q_temp = None if q_temp is None or not q_temp[0] else (float(q_temp[0]), int(q_temp[1]))
        self.gate, self.out_scale, self.own_kv = bool(gate), float(out_scale), bool(own_kv)
        self.gate_heads = gate == "head"
        self.sink_name, self.talk_name = sink_name, talk_name
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps else 0.0
        self.float_out = bool(float_out)
        self.qw = num_heads * dim
        self.kw = num_kv_heads * dim if own_kv else 0
        self.vw = num_kv_heads * vdim if own_kv else 0
        self.gw = (num_heads if self.gate_heads else num_heads * vdim) if gate else 0
        self.w_in = self.b_in = self.w_o = self.b_o = self.sinks = self.talk = None
        self._plan: Optional[PagedAttentionPlan] = None

    # ------------------------------------------------------------ tensors
    def _projections(self):
        out = [("q", self.qw)]
        if self.own_kv:
            out += [("k", self.kw), ("v", self.vw)]
        if self.gate:
            out.append(("g", self.gw))
        return out

    def param_specs(self) -> List[ParamSpec]:
        n, specs = self.names, []
        for key, rows in self._projections():
            specs.append(ParamSpec(n[key], (rows, self.hidden), MATRIX))
            if self.qkv_bias and key != "g":
                specs.append(ParamSpec(n[key] + self.suffix, (rows,), VECTOR))
        specs.append(ParamSpec(n["o"], (self.hidden, self.nh * self.vdim), MATRIX))
        if self.o_bias:
            specs.append(ParamSpec(n["o"] + self.suffix, (self.hidden,), VECTOR))
        if self.sink_name:
            specs.append(ParamSpec(self.sink_name, (self.nh,), VECTOR))
        if self.talk_name:
            specs.append(ParamSpec(self.talk_name, (self.nh, self.nh), VECTOR))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        mats, biases = [], []
        for key, rows in self._projections():
            w = tensors.pop(n[key])
            mats.append(w)
            if self.qkv_bias and key != "g":
                biases.append(tensors.pop(n[key] + self.suffix).to(torch.float32))
            else:
                biases.append(torch.zeros(rows, dtype=torch.float32, device=w.device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.b_in = torch.cat(biases, dim=0).contiguous() if self.qkv_bias else None
        self.w_o = tensors.pop(n["o"])
        self.b_o = tensors.pop(n["o"] + self.suffix) if self.o_bias else None
        if self.sink_name:
            self.sinks = tensors[self.sink_name].to(torch.float32).contiguous()
        if self.talk_name:
            self.talk = tensors[self.talk_name].to(torch.float32).contiguous()

    def param_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    # ------------------------------------------------------------ cache, plan
    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.nkv, self.dim, self.window, value_dim=self.vdim, keep_first=self.keep_first)

    def step_plan(self) -> StepPlan:
        # the paged attention's sorting of a step's tokens: portions in tiles, short ones and single tokens as items
        if self._plan is None:
            self._plan = PagedAttentionPlan()
        return self._plan

    # ------------------------------------------------------------ step
    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        n = h.shape[0]
        proj = ops.linear(h, self.w_in)
        q = torch.empty((n, self.qw), dtype=h.dtype, device=h.device)
        rot = self.qk_position
        rot_dims = rot.dims if rot is not None else 0
        temp = self.q_temp or (0.0, 1)
        ps = cache.page_size
        ops.gqa_prepare(proj, 0, self.qw, self.qw + self.kw, self.b_in, rot.inv_freq(h.device) if rot_dims else None,
                        rot_dims, temp[0], temp[1], q, cache.pool, cache.layer, ctx.positions, ctx.seq_of_token,
                        ctx.slots, cache.block_table, self.nh, self.nkv, self.dim, self.vdim, ps, ctx.status,
                        write_kv=self.own_kv and cache.writable, norm_eps=self.qk_norm_eps)
        o = torch.empty((n, self.nh * self.vdim), dtype=h.dtype, device=h.device)
        gate, gate_off = (proj, self.qw + self.kw + self.vw) if self.gate else (None, 0)
        sink = self.sinks if self.sinks is not None else self.sink
        if self.talk is not None or self.gate_heads:
            # every head's weights of a key meet before the values: the heads of a token are served together
            args = (cache.pool, cache.layer, o)
            tail = (self.nh, self.nkv, self.dim, self.vdim, ps, self.scale, self.window or 0, self.keep_first, self.talk,
                    self._sink_vector(h.device), gate, gate_off, self.gate_heads, self.out_scale)
            plan = ctx.plan(PagedAttentionPlan.name)
            rows = (ctx.positions, ctx.seq_of_token, ctx.slots, cache.block_table)
            tiles_ok = ops.talk_attention_tiles_applies(q, self.nh, self.nkv, self.dim, self.vdim)
            if h.dtype != torch.bfloat16 or (plan.n_tiles and not tiles_ok):
                ops.talk_attention_plain(q, *args, *rows, *tail, status=ctx.status)
            else:
                if plan.n_tiles:
                    ops.talk_attention_tiles(q, *args, plan.tiles, plan.n_tiles, self._plan.tile_rows, ctx.q_start,
                                             ctx.start_pos, ctx.slots, cache.block_table, *tail, status=ctx.status)
                if plan.n_items:
                    # the most keys a token of the step sees
                    cap = max(int(plan.max_item_kv), 1)
                    if self.window:
                        cap = min(cap, self.window + self.keep_first)
                    if ops.talk_attention_single_applies(q, self.nh, self.nkv, self.dim, self.vdim, cap):
                        scratch = ctx.scratch_f32(ops.talk_attention_single_scratch(plan.n_items, self.nh, cap))
                        ops.talk_attention_single(q, *args, *rows, *tail, scratch, cap, status=ctx.status,
                                                  items=plan.items, n_items=plan.n_items)
                    else:
                        ops.talk_attention_plain(q, *args, *rows, *tail, status=ctx.status, items=plan.items,
                                                 n_items=plan.n_items)
            return Delta(ops.linear(o, self.w_o, out_dtype=torch.float32 if self.float_out else None), self.b_o)
        consts = (self.nh, self.nkv, self.dim, self.vdim, ps, self.scale, self.window or 0, self.keep_first, sink,
                  gate, gate_off, self.out_scale)
        if ops.gqa_attention_fast_applies(q, self.nh, self.nkv, self.dim, self.vdim):
            plan = ctx.plan(PagedAttentionPlan.name)
            if plan.n_tiles:
                ops.gqa_attention_tiles(q, cache.pool, cache.layer, o, plan.tiles, plan.n_tiles, self._plan.tile_rows,
                                        ctx.q_start, ctx.start_pos, ctx.slots, cache.block_table, *consts,
                                        status=ctx.status)
            if plan.n_items:
                ops.gqa_attention_single(q, cache.pool, cache.layer, o, ctx.positions, ctx.seq_of_token, ctx.slots,
                                         cache.block_table, *consts, status=ctx.status, items=plan.items,
                                         n_items=plan.n_items)
        else:
            ops.gqa_attention_plain(q, cache.pool, cache.layer, o, ctx.positions, ctx.seq_of_token, ctx.slots,
                                    cache.block_table, *consts, status=ctx.status)
        return Delta(ops.linear(o, self.w_o, out_dtype=torch.float32 if self.float_out else None), self.b_o)

    def _sink_vector(self, device) -> Optional[torch.Tensor]:
        """The extra term's logit of every head for the kernels that take one per head (None: no extra term)."""
        if self.sinks is None and self.sink is not None:
            self.sinks = torch.full((self.nh,), self.sink, dtype=torch.float32, device=device)
        return self.sinks
