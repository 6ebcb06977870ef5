"""A selective state space (Mamba-2, state-space duality) in its recurrent form: a mixer with a matrix state."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, segment_plan
from ..registry import register_part
from .base import BuildContext, LayerBinding, Mixer, StateSpec, WeightSpec
from .short_conv import CausalConv
from .window_attention import pad8


class SelectiveStateSpace(Mixer):
    """``num_heads`` heads of ``v_dim`` inputs each (``inner = num_heads * v_dim``), a state of ``state_dim x v_dim`` per
    head (float32, zero at the start of a sequence), input and output matrices shared by the heads of a group (head h
    reads group ``h // (num_heads / groups)``):

    * ``W_in h`` is ``[z: inner | x: inner | B: groups * state_dim | C: groups * state_dim | dt: num_heads]``;
    * x, B and C together pass a short causal convolution per channel (``conv``, with bias ``conv.b``) and silu;
    * ``dt = softplus(dt + dt_bias)`` (no clamp); per head ``S <- exp(-exp(A_log) dt) S + dt B x^T``,
      ``y = S^T C + D x`` (y is read from the updated S);
    * the heads' y side by side times ``silu(z)``, then an RMS norm in ``norm_groups`` equal parts (each by its own root
      mean square, ``eps`` inside the root) times ``norm`` (gated first, normed after); then ``W_o``.

    Tensor names below the prefix: ``in, o`` (stored (out, in)), ``conv, conv.b``, ``dt_bias, A_log, D``, ``norm``.  On
    the device the input projection's columns lie as ``C | B | x | z | dt`` (what the recurrence's kernel takes as
    queries, keys and values comes first and in its order).  The step size, the decay, the state, the recurrence, the
    gate and the norm are 32-bit.  The state of a request is S of every head followed by the convolution's last inputs."""

    graph_safe = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, v_dim: int, state_dim: int, groups: int, norm_groups: int, conv_taps: int,
                 eps: float, prefix: str = ""):
        super().__init__(prefix)
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads are not a multiple of {groups} groups")
        self.width, self.num_heads, self.v_dim, self.state_dim, self.groups = width, num_heads, v_dim, state_dim, groups
        self.inner = num_heads * v_dim
        if norm_groups <= 0 or self.inner % norm_groups:
            raise ValueError(f"a norm over {self.inner} elements in {norm_groups} groups")
        self.norm_groups, self.eps = norm_groups, float(eps)
        self.gn = groups * state_dim
        self.nc = 2 * self.gn + self.inner                   # channels that pass the convolution
        self.conv = CausalConv([self.nc], conv_taps, ["conv"], prefix=prefix, silu=True, bias_name="conv.b")
        # the convolution's tensors are stored in the order x | B | C; the rows it is given hold C | B | x
        self.conv.order(torch.cat([torch.arange(self.inner + self.gn, self.inner + 2 * self.gn),
                                   torch.arange(self.inner, self.inner + self.gn), torch.arange(0, self.inner)]))
        self.state_matrix = num_heads * state_dim * v_dim
        self.z_at = pad8(self.nc)
        self.dt_at = self.z_at + pad8(self.inner)
        self.cols = self.dt_at + pad8(num_heads)
        self.w_in = self.w_o = self.a_log = self.dt_bias = self.skip = self.norm_w = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None, mixer: Optional[dict] = None):
        m = mixer if mixer is not None else cfg.layers[layer_index]["mixer"]
        return cls(cfg.hidden_size, m["heads"], m["vdim"], m["state"], m["groups"], m.get("norm_groups", 1), m["conv"],
                   cfg.rms_norm_eps, prefix=prefix)

    def children(self):
        return (self.conv,)

    def step_planners(self):
        return (segment_plan.planner(),)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.state_matrix + self.conv.state_floats,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h = self.num_heads
        return {"in": WeightSpec((2 * self.inner + 2 * self.gn + h, self.width)),
                "dt_bias": WeightSpec((h,), init="uniform", lo=-2.0, hi=1.0),
                "A_log": WeightSpec((h,), init="uniform", lo=-1.0, hi=1.0), "D": WeightSpec((h,), init="ones_normal"),
                "norm": WeightSpec((self.inner,), init="ones_normal"), "o": WeightSpec((self.width, self.inner))}

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        inner, gn, h = self.inner, self.gn, self.num_heads
        stored = tensors[p + "in"].to(ctx.dtype)             # rows: z | x | B | C | dt
        z, x = stored[:inner], stored[inner:2 * inner]
        b, c = stored[2 * inner:2 * inner + gn], stored[2 * inner + gn:2 * inner + 2 * gn]
        dt = stored[2 * inner + 2 * gn:]
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        w[:, :self.nc] = torch.cat([c, b, x], dim=0).t()
        w[:, self.z_at:self.z_at + inner] = z.t()
        w[:, self.dt_at:self.dt_at + h] = dt.t()
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.a_log = tensors[p + "A_log"].to(**f32).contiguous()
        self.dt_bias = tensors[p + "dt_bias"].to(**f32).contiguous()
        self.skip = tensors[p + "D"].to(**f32).contiguous()
        self.norm_w = tensors[p + "norm"].to(**f32).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n, h = x.shape[0], self.num_heads
        proj = ops.gemm(x, self.w_in)
        cbx = self.conv.forward(proj[:, :self.nc], step, binding.state[:, self.state_matrix:])
        raw = ops.state_space_scan(cbx, proj[:, self.dt_at:self.dt_at + h], self.a_log, self.dt_bias, binding.state,
                                   step.row_slot, step.row_last, h, self.groups, self.state_dim, self.v_dim,
                                   requests=len(step.segments), segments=step.plan(segment_plan.planner()))
        out = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        ops.skip_gate_group_norm(raw, cbx[:, 2 * self.gn:], self.skip, proj[:, self.z_at:self.z_at + self.inner],
                                 self.norm_w, self.norm_groups, self.eps, out, step.row_slot, h, self.v_dim)
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "selective_state_space", SelectiveStateSpace)
