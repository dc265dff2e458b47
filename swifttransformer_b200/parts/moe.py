"""A routed mixture of gated feed-forward experts, with an optional shared expert.

    z = W_r h  (float)           s = softmax(z) over all experts
    the ``top`` experts with the largest s are chosen; their weights are their s (divided by their sum only with
    ``renormalise``)
    out = sum over the chosen e of s_e * down_e(act(gate_e h) * (up_e h))
          + sigmoid(w_sg . h) * down_s(act(gate_s h) * (up_s h))          the shared expert, for every token

With ``limit`` the experts are clamped gated units instead: g = min(gate_e h, limit), u = clamp(up_e h, -limit, limit),
down_e(g * sigmoid(alpha * g) * (u + shift)).

On the device the step's (token, choice) items are grouped by expert (``ops.moe_sort``), two grouped products run
over the groups (gate|up with the activation in the epilogue, then down), and one kernel forms the weighted sums and
adds the gated shared expert, in float.  Nothing comes back to the host, so steps are recorded like any others.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, ParamSpec
from .base import FEED_FORWARDS, Delta, FeedForward, Part


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """expert_names: per expert {"gate", "up", "down"} tensor names; router_name: [experts, hidden] (kept in float);
    shared: a feed-forward part for every token or None, with shared_gate_name ([1, hidden] or [hidden], float) the
    weight of its sigmoid gate (None: the shared expert is added as it is)."""

    def __init__(self, hidden: int, inner: int, num_experts: int, top: int, activation: str,
                 expert_names: List[Dict[str, str]], router_name: str, shared: Optional[FeedForward] = None,
                 shared_gate_name: Optional[str] = None, renormalise: bool = False, limit: Optional[float] = None,
                 alpha: float = 1.0, shift: float = 0.0):
        self.limit, self.alpha, self.shift = (float(limit) if limit else None), float(alpha), float(shift)
        if activation not in ops.ACT_CODES:
            raise ValueError(f"activation '{activation}' is not supported ({', '.join(ops.ACT_CODES)})")
        if len(expert_names) != num_experts or not 1 <= top <= num_experts:
            raise ValueError("a mixture needs names for every expert and 1 <= top <= experts")
        self.hidden, self.inner, self.n_experts, self.top, self.activation = hidden, inner, num_experts, top, activation
        self.expert_names, self.router_name = expert_names, router_name
        self.shared, self.shared_gate_name, self.renormalise = shared, shared_gate_name, renormalise
        self.w_router = self.w_gu = self.w_down = self.w_sg = None

    def children(self) -> List[Part]:
        return [self.shared] if self.shared is not None else []

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.router_name, (self.n_experts, self.hidden), VECTOR)]
        for n in self.expert_names:
            specs += [ParamSpec(n["gate"], (self.inner, self.hidden), MATRIX),
                      ParamSpec(n["up"], (self.inner, self.hidden), MATRIX),
                      ParamSpec(n["down"], (self.hidden, self.inner), MATRIX)]
        if self.shared is not None and self.shared_gate_name:
            specs.append(ParamSpec(self.shared_gate_name, (1, self.hidden), VECTOR))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_router = tensors[self.router_name]
        # [experts, 2 * inner, hidden]: an expert's gate rows, then its up rows; [experts, hidden, inner]
        self.w_gu = torch.stack([torch.cat([tensors.pop(n["gate"]), tensors.pop(n["up"])], dim=0)
                                 for n in self.expert_names]).contiguous()
        self.w_down = torch.stack([tensors.pop(n["down"]) for n in self.expert_names]).contiguous()
        if self.shared is not None and self.shared_gate_name:
            self.w_sg = tensors[self.shared_gate_name].reshape(-1).contiguous()

    def forward(self, h: torch.Tensor, ctx: Any) -> Delta:
        experts, weights, gate = ops.moe_route(h, self.w_router, self.top, ctx.positions, self.w_sg, self.renormalise)
        order = ops.moe_sort(experts, self.n_experts)
        if self.limit is not None:
            # gate | up of every item as the product leaves them, then the clamped unit over the rows
            u = ops.gated_clamped_act(ops.gemm_experts(h, self.w_gu, order, gather=True), None, self.limit, self.alpha,
                                      self.shift)
        else:
            u = ops.gemm_experts(h, self.w_gu, order, gather=True, gated=True, act=self.activation)
        y = ops.gemm_experts(u, self.w_down, order, gather=False)
        shared = None
        if self.shared is not None:
            s = self.shared.forward(h, ctx)
            assert s.bias is None and s.parts is None
            shared = s.value
            if gate is None:
                gate = torch.ones((h.shape[0],), dtype=torch.float32, device=h.device)
        return Delta(ops.moe_combine(y, order, weights, shared, gate, out_dtype=torch.float32))

    def param_bytes(self) -> int:
        """What a step reads at most: every expert's matrices (a step of few tokens reads only the chosen ones)."""
        return (self.w_gu.numel() + self.w_down.numel()) * self.w_gu.element_size() + self.w_router.numel() * 4
