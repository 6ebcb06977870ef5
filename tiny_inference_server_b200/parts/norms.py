"""Norms."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import BuildContext, Norm, WeightSpec


class RMSNormL2(Norm):
    """``y = x * sqrt(width) / (||x||_2 + eps) * scale`` in float32, eps added to the L2
    norm itself (upstream ``rms_norm``, main_models_new.py:31-42, where eps is the
    constant 2e-8; here it is a parameter)."""

    def __init__(self, width: int, eps: float, prefix: str = "", weight_name: str = "scale"):
        super().__init__(prefix)
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.scale: Optional[torch.Tensor] = None
        self.out_dtype = torch.float32

    @classmethod
    def from_config(cls, cfg, prefix: str):
        return cls(cfg.hidden_size, cfg.rms_norm_eps, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), init="ones_normal")}

    def load(self, tensors, ctx: BuildContext) -> None:
        self.scale = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.out_dtype = ctx.dtype

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], delta_norm=None) -> torch.Tensor:
        out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.scale, self.eps, out, delta_norm=delta_norm)

    def forward(self, residual: torch.Tensor) -> torch.Tensor:
        return self.add_norm(residual, None)

    def as_delta_norm(self):
        """(weight, eps, kind of factor): this norm applied to an update on its way into the stream."""
        return (self.scale, self.eps, "l2_eps")

    def sink(self, values: torch.Tensor):
        # the factor of a row, sqrt(width) / (||row|| + eps), is what the products apply themselves
        return ops.ResidualSink(values, self.scale, self.eps, norm=self)


class RMSNormMeanEps(Norm):
    """``y = x / sqrt(mean(x^2) + eps) * (offset + w)`` in float32, eps inside the root.  ``offset`` 1: the
    stored tensor is the weight's distance from one; 0: it is the weight.  ``keep_f32``: the result is float32
    whatever the compute dtype."""

    def __init__(self, width: int, eps: float, prefix: str = "", weight_name: str = "weight", offset: float = 0.0,
                 keep_f32: bool = False):
        super().__init__(prefix)
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.offset = float(offset)
        self.keep_f32 = keep_f32                  # the result stays in 32-bit (a norm that makes the residual stream)
        self.scale: Optional[torch.Tensor] = None
        self.out_dtype = torch.float32

    @classmethod
    def from_config(cls, cfg, prefix: str):
        return cls(cfg.hidden_size, cfg.rms_norm_eps, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), init="normal" if self.offset else "ones_normal")}

    def load(self, tensors, ctx: BuildContext) -> None:
        w = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=torch.float32)
        self.scale = (w + self.offset).contiguous()
        self.out_dtype = torch.float32 if self.keep_f32 else ctx.dtype

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], delta_norm=None) -> torch.Tensor:
        out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.scale, self.eps, out, kind="mean_eps", delta_norm=delta_norm)

    def forward(self, residual: torch.Tensor) -> torch.Tensor:
        return self.add_norm(residual, None)

    def as_delta_norm(self):
        """(weight, eps, kind of factor): this norm applied to an update on its way into the stream."""
        return (self.scale, self.eps, "mean_eps")

    def sink(self, values: torch.Tensor):
        return ops.ResidualSink(values, self.scale, self.eps, norm=self, kind="mean_eps")


class RMSNormOnePlus(RMSNormMeanEps):
    """``RMSNormMeanEps`` whose tensor holds the weight minus one: ``x / sqrt(mean(x^2) + eps) * (1 + w)``."""

    def __init__(self, width: int, eps: float, prefix: str = "", weight_name: str = "weight"):
        super().__init__(width, eps, prefix=prefix, weight_name=weight_name, offset=1.0)


class RMSNormScalar(RMSNormMeanEps):
    """``x / sqrt(mean(x^2) + eps) * g`` with ONE number ``g`` for all coordinates (the tensor has no dimensions).  On
    the device the number is spread over the width, so that the kernels of the other norms serve."""

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((), init="ones_normal")}

    def load(self, tensors, ctx: BuildContext) -> None:
        g = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=torch.float32).reshape(())
        self.scale = (g + self.offset).expand(self.width).contiguous()
        self.out_dtype = torch.float32 if self.keep_f32 else ctx.dtype


class RMSNormGrouped(Norm):
    """The RMS norm in groups: the vector is cut into ``groups`` equal consecutive parts, every part is divided by its own
    ``sqrt(mean(part^2) + eps)`` (eps inside the root), and the whole is multiplied by ``w`` (one weight per element);
    32-bit.  ``groups`` 1 is the plain norm.

    Two things that a layer whose sublayers read the same stream wants of its norms, each one kernel:
    ``add_norm(residual, delta, delta_b=...)`` adds two pending updates before it normalises, and
    ``add_norm_pair(residual, delta, delta_b, other)`` also writes the output of a second norm of the same groups and eps
    (``other``), whose factors are the same."""

    def __init__(self, width: int, groups: int, eps: float, prefix: str = "", weight_name: str = "weight"):
        super().__init__(prefix)
        if groups <= 0 or width % groups:
            raise ValueError(f"a norm over {width} elements in {groups} groups")
        self.width, self.groups, self.eps = width, groups, float(eps)
        self.weight_name = weight_name
        self.scale: Optional[torch.Tensor] = None
        self.out_dtype = torch.float32

    @classmethod
    def from_config(cls, cfg, prefix: str):
        return cls(cfg.hidden_size, cfg.norm_groups, cfg.rms_norm_eps, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.width,), init="ones_normal")}

    def load(self, tensors, ctx: BuildContext) -> None:
        self.scale = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.out_dtype = ctx.dtype

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], delta_norm=None, delta_b=None) -> torch.Tensor:
        if delta_norm is not None:
            raise ValueError("the norm in groups takes updates as they are")
        out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        ops.group_norm(residual, delta, delta_b, self.groups, self.eps, self.scale, out)
        return out

    def add_norm_pair(self, residual: torch.Tensor, delta: Optional[torch.Tensor], delta_b: Optional[torch.Tensor],
                      other: "RMSNormGrouped"):
        """(this norm's output, ``other``'s output) of ``residual + delta + delta_b``, which stays in ``residual``."""
        if other.groups != self.groups or other.eps != self.eps or other.out_dtype != self.out_dtype:
            raise ValueError("a pair of norms shares groups, eps and output type")
        a = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        b = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        ops.group_norm(residual, delta, delta_b, self.groups, self.eps, self.scale, a, other.scale, b)
        return a, b

    def forward(self, residual: torch.Tensor) -> torch.Tensor:
        return self.add_norm(residual, None)

    def in_place(self, values: torch.Tensor) -> torch.Tensor:
        """``values`` (float32) replaced by its norm: a norm that makes the residual stream."""
        ops.group_norm(values, None, None, self.groups, self.eps, self.scale, None, in_place=True)
        return values


register_part("norm", "rmsnorm_grouped", RMSNormGrouped)
register_part("norm", "rmsnorm_l2", RMSNormL2)
register_part("norm", "rmsnorm_mean_eps", RMSNormMeanEps)
register_part("norm", "rmsnorm_one_plus", RMSNormOnePlus)
register_part("norm", "rmsnorm_scalar", RMSNormScalar)
