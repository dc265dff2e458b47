"""Two mixers side by side: both read the same input, and their results are added.

    out = a * left(h) + b * right(h)

The weights a and b are not applied here: every mixer that can stand in this place takes an ``out_scale`` that its
last kernel before the output projection applies (in float, before the result is rounded to the storage type),
so the sum needs no pass of its own: the left mixer's result (storage type) and the right one's (float32) are left
pending together, and the next norm kernel adds both to the float residual rows.  The cache entry of the pair is
the pair of its members' needs.

With ``norm_names`` each member's result is first RMS-normed over the model width with a weight vector of its own,

    out = a * w_l * left(h) / rms(left(h)) + b * w_r * right(h) / rms(right(h)),

in one kernel that leaves the sum as float32 rows (``weights`` = (a, b)); the members then keep ``out_scale`` 1.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from .. import ops
from ..weights.spec import GAIN, ParamSpec
from .base import MIXERS, Delta, Mixer, Part


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    def __init__(self, left: Mixer, right: Mixer, norm_names: Optional[Tuple[str, str]] = None, width: int = 0,
                 eps: float = 1e-5, weights: Tuple[float, float] = (1.0, 1.0)):
        if not getattr(right, "float_out", False):
            raise ValueError("the right mixer of a pair must leave its result in float32 (float_out)")
        if norm_names is not None and width <= 0:
            raise ValueError("a pair with output norms needs the model width")
        self.left, self.right = left, right
        self.norm_names, self.width, self.eps = (tuple(norm_names) if norm_names else None), int(width), float(eps)
        self.weights = (float(weights[0]), float(weights[1]))
        self.w_left = self.w_right = None

    def param_specs(self) -> List[ParamSpec]:
        if self.norm_names is None:
            return []
        return [ParamSpec(name, (self.width,), GAIN) for name in self.norm_names]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.norm_names is not None:
            self.w_left, self.w_right = (tensors[name] for name in self.norm_names)

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def children(self) -> List[Part]:
        return [self.left, self.right]

    def cache_spec(self):
        return (self.left.cache_spec(), self.right.cache_spec())

    def step_plan(self):
        # (at most one member has a plan of its own kind; both would share it by name anyway)
        return self.left.step_plan() or self.right.step_plan()

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        a = self.left.forward(h, ctx, cache[0])
        b = self.right.forward(h, ctx, cache[1])
        assert a.parts is None and b.bias is None and b.parts is None
        assert b.value.dtype == torch.float32 and b.value.is_contiguous()
        if self.norm_names is not None:
            assert a.bias is None
            return Delta(ops.norm_pair_sum(a.value, self.w_left, self.weights[0], b.value, self.w_right,
                                           self.weights[1], self.eps, ctx.positions))
        return Delta(a.value, a.bias, b.value.unsqueeze(0))

    def param_bytes(self) -> int:
        return self.left.param_bytes() + self.right.param_bytes()
