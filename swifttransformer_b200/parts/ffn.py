"""The dense feed-forward: z = act(h fc1^T + b1) fc2^T + b2.

Reference: ``st::layer::ffn`` (src/csrc/layer/ffn.cc:49-126): fc1 product (71-80),
fused bias + activation (85-92), fc2 product (96-105), bias (124).  The second
bias travels with the result so the next norm kernel adds it with the residual.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, ParamSpec
from .base import FEED_FORWARDS, Delta, FeedForward


@FEED_FORWARDS.register("dense")
class DenseFFN(FeedForward):
    def __init__(self, hidden: int, inner: int, activation: str, fc1_name: str, fc2_name: str, bias: bool = True):
        if activation not in ops.ACT_CODES:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(ops.ACT_CODES)})")
        self.hidden, self.inner, self.activation, self.bias = hidden, inner, activation, bias
        self.fc1_name, self.fc2_name = fc1_name, fc2_name
        self.w1 = self.b1 = self.w2 = self.b2 = self.b1_bf16 = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.fc1_name + ".weight", (self.inner, self.hidden), MATRIX),
                 ParamSpec(self.fc2_name + ".weight", (self.hidden, self.inner), MATRIX)]
        if self.bias:
            specs += [ParamSpec(self.fc1_name + ".bias", (self.inner,), VECTOR),
                      ParamSpec(self.fc2_name + ".bias", (self.hidden,), VECTOR)]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w1, self.w2 = tensors[self.fc1_name + ".weight"], tensors[self.fc2_name + ".weight"]
        if self.bias:
            self.b1, self.b2 = tensors[self.fc1_name + ".bias"], tensors[self.fc2_name + ".bias"]
            if self.w1.dtype == torch.bfloat16:
                # lets the library product add the bias (and apply ReLU) in its epilogue
                self.b1_bf16 = ops.lossless_bf16(self.b1)

    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        u = ops.linear(h, self.w1, self.b1, self.activation, bias_bf16=self.b1_bf16)
        if u.shape[0] > ops.SKINNY_MAX_ROWS and ops.linear_parts_slices(u.shape[0], self.w2) > 1:
            # fc2 for this many tokens is cut over k: its slices' sums are left for the next norm kernel
            return Delta(None, self.b2, ops.linear_parts(u, self.w2))
        return Delta(ops.linear(u, self.w2), self.b2)

    def forward_into_residual(self, x: torch.Tensor, norm: Any, ctx: Any, pending: Optional[Delta] = None) -> Any:
        """x <- (x + pending) + ffn(norm(x + pending)) for a step of a few tokens: norm (which adds what is pending)
        and fc1 + bias + activation; then fc2 + bias + residual sum in one kernel, or, where that kernel would cut
        fc2 over k, the slices' sums left as a Delta for the next norm kernel to add."""
        if norm.kind not in ops.NORM_CODES or not ops.fused_norm_applies(x.shape[0], self.hidden, self.w1):
            return False
        if self.inner % 8 or (pending is not None and ops.FUSE_NORM):
            return False
        u = ops.norm_linear(x, norm.kind, norm.gamma, norm.beta, norm.eps, self.w1, self.b1, self.activation,
                            delta=pending.value if pending else None, delta_bias=pending.bias if pending else None,
                            parts=pending.parts if pending else None)
        if not ops.FUSE_NORM and ops.linear_parts_slices(x.shape[0], self.w2) > 1 and self.inner > ops.UNCUT_MAX_INNER:
            return Delta(None, self.b2, ops.linear_parts(u, self.w2))
        ops.linear_add(u, self.w2, self.b2, x)
        return True

    def param_bytes(self) -> int:
        return (self.w1.numel() + self.w2.numel()) * self.w1.element_size()


@FEED_FORWARDS.register("gated")
class GatedFFN(FeedForward):
    """z = down(act(gate h) * (up h)), no biases.  The gate and up matrices are stacked at load time so that one
    product gives both; ``activation`` is any of ops.ACT_CODES (the tanh form of GELU, SiLU, ...).  ``float_out``:
    the down product leaves its float sums as they are (a block that adds two sub-layers' results takes them so)."""

    def __init__(self, hidden: int, inner: int, activation: str, gate_name: str, up_name: str, down_name: str,
                 float_out: bool = False):
        self.float_out = float_out
        if activation not in ops.ACT_CODES:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(ops.ACT_CODES)})")
        self.hidden, self.inner, self.activation = hidden, inner, activation
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gu = self.w_down = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.gate_name, (self.inner, self.hidden), MATRIX),
                ParamSpec(self.up_name, (self.inner, self.hidden), MATRIX),
                ParamSpec(self.down_name, (self.hidden, self.inner), MATRIX)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gu = torch.cat([tensors.pop(self.gate_name), tensors.pop(self.up_name)], dim=0).contiguous()
        self.w_down = tensors[self.down_name]

    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        u = ops.gated_act(ops.linear(h, self.w_gu), self.activation)
        return Delta(ops.linear(u, self.w_down, out_dtype=torch.float32 if self.float_out else None))

    def param_bytes(self) -> int:
        return (self.w_gu.numel() + self.w_down.numel()) * self.w_gu.element_size()


@FEED_FORWARDS.register("gated_clamped")
class ClampedGatedFFN(FeedForward):
    """z = down(g * sigmoid(alpha * g) * (u + shift)) + b_down with g = min(gate h + b_gate, limit) and
    u = clamp(up h + b_up, -limit, limit).  The gate and up matrices are stacked at load time so that one product
    gives both; their biases, the limits and the unit are one kernel.  ``bias``: whether the three projections have
    biases (a projection's bias is its name + ``bias_suffix``)."""

    def __init__(self, hidden: int, inner: int, limit: float, gate_name: str, up_name: str, down_name: str,
                 alpha: float = 1.0, shift: float = 0.0, bias: bool = True, bias_suffix: str = ".b"):
        self.hidden, self.inner, self.limit, self.alpha, self.shift = hidden, inner, float(limit), float(alpha), float(shift)
        self.gate_name, self.up_name, self.down_name, self.bias, self.suffix = gate_name, up_name, down_name, bias, bias_suffix
        self.w_gu = self.b_gu = self.w_down = self.b_down = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.gate_name, (self.inner, self.hidden), MATRIX),
                 ParamSpec(self.up_name, (self.inner, self.hidden), MATRIX),
                 ParamSpec(self.down_name, (self.hidden, self.inner), MATRIX)]
        if self.bias:
            specs += [ParamSpec(self.gate_name + self.suffix, (self.inner,), VECTOR),
                      ParamSpec(self.up_name + self.suffix, (self.inner,), VECTOR),
                      ParamSpec(self.down_name + self.suffix, (self.hidden,), VECTOR)]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gu = torch.cat([tensors.pop(self.gate_name), tensors.pop(self.up_name)], dim=0).contiguous()
        self.w_down = tensors[self.down_name]
        if self.bias:
            self.b_gu = torch.cat([tensors.pop(self.gate_name + self.suffix), tensors.pop(self.up_name + self.suffix)],
                                  dim=0).contiguous()
            self.b_down = tensors[self.down_name + self.suffix]

    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        u = ops.gated_clamped_act(ops.linear(h, self.w_gu), self.b_gu, self.limit, self.alpha, self.shift)
        return Delta(ops.linear(u, self.w_down), self.b_down)

    def param_bytes(self) -> int:
        return (self.w_gu.numel() + self.w_down.numel()) * self.w_gu.element_size()


@FEED_FORWARDS.register("dense_xielu")
class XieluFFN(FeedForward):
    """z = down(act(up h)), no biases, with the two-sided activation

        act(z) = a_p z^2 + z / 2                    for z > 0
               = a_n (exp(z) - 1 - z) + z / 2       for z <= 0,     a_p = softplus(p),  a_n = shift + softplus(q),

    whose two numbers (p, q) are the tensor ``act_name`` [2]; ``shift`` is the constant added to softplus(q).  The
    two factors are formed once, in double precision, when the weights are bound."""

    def __init__(self, hidden: int, inner: int, up_name: str, down_name: str, act_name: str, shift: float = 0.5,
                 float_out: bool = False):
        self.hidden, self.inner, self.shift, self.float_out = hidden, inner, float(shift), bool(float_out)
        self.up_name, self.down_name, self.act_name = up_name, down_name, act_name
        self.w_up = self.w_down = None
        self.alpha_pos = self.alpha_neg = 0.0

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.up_name, (self.inner, self.hidden), MATRIX),
                ParamSpec(self.down_name, (self.hidden, self.inner), MATRIX),
                ParamSpec(self.act_name, (2,), VECTOR)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = tensors[self.up_name], tensors[self.down_name]
        p, q = (float(v) for v in tensors[self.act_name].to(torch.float64).cpu())
        softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))
        self.alpha_pos, self.alpha_neg = softplus(p), self.shift + softplus(q)

    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        u = ops.xielu(ops.linear(h, self.w_up), self.alpha_pos, self.alpha_neg)
        return Delta(ops.linear(u, self.w_down, out_dtype=torch.float32 if self.float_out else None))

    def param_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_up.element_size()
