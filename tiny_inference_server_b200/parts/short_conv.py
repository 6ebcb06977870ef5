"""A short causal convolution over time on each channel, with per-request state."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..kernels import ops
from .base import BuildContext, Part, StateSpec, WeightSpec


class CausalConv(Part):
    """``y_t = [x_t +] [b +] sum_j w[:, j] * x_(t - taps + 1 + j)``, optionally through silu: the last column of
    ``w`` weighs the current position, inputs before the start of a sequence are zero; ``bias_name``: a tensor
    ``(channels,)`` that is added (None: no bias).  The last
    ``taps - 1`` inputs of a request are its state (float32, ``state_floats`` per request), so that a step
    may bring any part of a sequence, down to one token.

    ``weight_names``: the tensors ``(channels_i, taps)`` whose channels lie one after the other in the
    rows this part is given (the projections of a mixer, convolved in one launch).  Used alone in front
    of a mixer (``residual=True``: the block's input filter) or inside a mixer on its projections."""

    def __init__(self, channels: Sequence[int], taps: int, weight_names: Sequence[str], prefix: str = "",
                 residual: bool = False, silu: bool = False, bias_name: Optional[str] = None):
        super().__init__(prefix)
        if not (1 <= taps <= 16):
            raise ValueError(f"a short convolution of {taps} taps: the kernel takes 1..16")
        self.sections = list(channels)
        self.channels = sum(self.sections)
        self.taps = taps
        self.weight_names = list(weight_names)
        self.residual = residual
        self.silu = silu
        self.bias_name = bias_name
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.channel_order: Optional[torch.Tensor] = None

    @property
    def state_floats(self) -> int:
        return (self.taps - 1) * self.channels

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((max(1, self.state_floats),), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {name: WeightSpec((c, self.taps)) for name, c in zip(self.weight_names, self.sections)}
        if self.bias_name is not None:
            specs[self.bias_name] = WeightSpec((self.channels,))
        return specs

    def order(self, index: torch.Tensor) -> None:
        """Channel ``i`` of the rows this part is given is channel ``index[i]`` of the stored tensors (a mixer that lays
        its projections out in another order than the convolution's tensors).  Called before or after ``load``."""
        self.channel_order = index.clone()
        if self.weight is not None:
            self._reorder()

    def _reorder(self) -> None:
        index = self.channel_order.to(self.weight.device)
        self.weight = self.weight.index_select(1, index).contiguous()
        if self.bias is not None:
            self.bias = self.bias.index_select(0, index).contiguous()

    def load(self, tensors, ctx: BuildContext) -> None:
        w = torch.cat([tensors[self.prefix + name].to(torch.float32) for name in self.weight_names], dim=0)
        self.weight = w.t().contiguous().to(ctx.device)            # tap by tap: (taps, channels)
        if self.bias_name is not None:
            self.bias = tensors[self.prefix + self.bias_name].to(device=ctx.device, dtype=torch.float32).contiguous()
        if self.channel_order is not None:
            self._reorder()

    def forward(self, x: torch.Tensor, step, state: torch.Tensor) -> torch.Tensor:
        """``x`` (n, channels), row stride free; ``state`` (slots, >= state_floats) float32."""
        out = torch.empty((x.shape[0], self.channels), dtype=x.dtype, device=x.device)
        return ops.causal_conv(x, self.weight, state, out, step.row_slot, step.row_last, residual=self.residual,
                               silu=self.silu, bias=self.bias)
