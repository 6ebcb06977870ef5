"""Two mixers side by side: both read the same input and their results are added with a weight each."""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import KVSpec, LayerBinding, Mixer, StateSpec


class SideBySide(Mixer):
    """``left_scale * left(h) + right_scale * right(h)`` for two mixers ``left`` and ``right`` of any kind; the sum is
    formed in 32-bit.  At most one of the two may keep keys and values in the paged cache (the block has one cache
    plane); both may keep fixed-size state: the block's state is then the left one's followed by the right one's."""

    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0, prefix: str = ""):
        super().__init__(prefix)
        if left.kv_spec() is not None and right.kv_spec() is not None:
            raise ValueError("of two mixers side by side only one can keep keys and values")
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.graph_safe = left.graph_safe and right.graph_safe
        specs = [left.state_spec(), right.state_spec()]
        self._floats = [0 if s is None else int(torch.Size(s.shape).numel()) for s in specs]
        for s in specs:
            if s is not None and s.dtype != torch.float32:
                raise ValueError("states side by side are float32")

    def children(self):
        return (self.left, self.right)

    def kv_spec(self) -> Optional[KVSpec]:
        return self.left.kv_spec() or self.right.kv_spec()

    def state_spec(self) -> Optional[StateSpec]:
        total = sum(self._floats)
        return StateSpec((total,), torch.float32) if total else None

    def step_planners(self):
        return tuple(self.left.step_planners()) + tuple(self.right.step_planners())

    def forward(self, x, step, binding: LayerBinding):
        lb = rb = binding
        if self._floats[0] and self._floats[1]:
            lb = dataclasses.replace(binding, state=binding.state[:, :self._floats[0]])
            rb = dataclasses.replace(binding, state=binding.state[:, self._floats[0]:])
        a = self.left.forward(x, step, lb)
        b = self.right.forward(x, step, rb)
        return ops.scaled_sum(a, self.left_scale, b, self.right_scale)


register_part("mixer", "side_by_side", SideBySide)
