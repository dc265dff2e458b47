"""Two mixers side by side: both read the same input, and their results are added.

    out = a * left(h) + b * right(h)

The weights a and b are not applied here: every mixer that can stand in this place takes an ``out_scale`` that its
last kernel before the output projection applies (in float, before the result is rounded to the storage type),
so the sum needs no pass of its own: the left mixer's result (storage type) and the right one's (float32) are left
pending together, and the next norm kernel adds both to the float residual rows.  The cache entry of the pair is
the pair of its members' needs.
"""
from __future__ import annotations

from typing import Any, List

import torch

from .base import MIXERS, Delta, Mixer, Part


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    def __init__(self, left: Mixer, right: Mixer):
        if not getattr(right, "float_out", False):
            raise ValueError("the right mixer of a pair must leave its result in float32 (float_out)")
        self.left, self.right = left, right

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
        return Delta(a.value, a.bias, b.value.unsqueeze(0))

    def param_bytes(self) -> int:
        return self.left.param_bytes() + self.right.param_bytes()
