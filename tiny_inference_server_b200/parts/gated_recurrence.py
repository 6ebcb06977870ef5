"""A recurrent mixer whose forget gate also decides what is written (HGRN2)."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops, segment_plan
from ..registry import register_part
from .base import BuildContext, LayerBinding, Mixer, StateSpec, WeightSpec
from .window_attention import pad8


class ForgetGateRecurrence(Mixer):
    """Per head a state ``S`` (``k_dim x v_dim``, float32, zero at the start of a sequence):

    * ``q = silu(Wq h)`` (``num_heads`` heads of ``k_dim``), ``v = Wv h`` (heads of ``v_dim``);
    * the forget gate per head and key channel, ``f = lower + (1 - lower) * sigmoid(Wf h + f.b)``, with a lower bound
      ``lower`` per channel;
    * ``S <- diag(f) S + (1 - f) v^T;  o = S^T q`` (o is read from the updated S): one minus the gate stands where
      linear attention has a key, there is no key projection and no other scale;
    * every head's ``o`` is divided by its root mean square over ``v_dim`` (``eps`` inside the root) and multiplied by
      ``norm`` (``v_dim`` weights shared by the heads); then ``Wo``.

    Tensor names below the prefix: ``q, f, v, o`` (stored (out, in)), ``f.b``, ``lower``, ``norm``.  The gate, the
    state, the recurrence and the norm are 32-bit; the state lives in the cache manager's state slots."""

    graph_safe = True

    def __init__(self, width: int, num_heads: int, k_dim: int, v_dim: int, eps: float, prefix: str = ""):
        super().__init__(prefix)
        self.width, self.num_heads, self.k_dim, self.v_dim = width, num_heads, k_dim, v_dim
        self.eps = float(eps)
        self.nq = num_heads * k_dim
        self.nv = num_heads * v_dim
        self.f_at = pad8(self.nq + self.nv)                 # columns of the fused input projection: q | v | f
        self.cols = self.f_at + pad8(self.nq)
        self.w_in = self.w_o = self.f_bias = self.lower = self.norm_w = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None):
        m = cfg.layers[layer_index]["mixer"]
        return cls(cfg.hidden_size, m["heads"], m["dim"], m["vdim"], cfg.rms_norm_eps, prefix=prefix)

    def step_planners(self):
        return (segment_plan.planner(),)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads * self.k_dim * self.v_dim,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"q": WeightSpec((self.nq, self.width)), "f": WeightSpec((self.nq, self.width)),
                "f.b": WeightSpec((self.nq,)), "lower": WeightSpec((self.nq,), init="uniform", lo=0.0, hi=0.9),
                "v": WeightSpec((self.nv, self.width)), "norm": WeightSpec((self.v_dim,), init="ones_normal"),
                "o": WeightSpec((self.width, self.nv))}

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        w[:, :self.nq] = tensors[p + "q"].to(ctx.dtype).t()
        w[:, self.nq:self.nq + self.nv] = tensors[p + "v"].to(ctx.dtype).t()
        w[:, self.f_at:self.f_at + self.nq] = tensors[p + "f"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.f_bias = tensors[p + "f.b"].to(**f32).contiguous()
        self.lower = tensors[p + "lower"].to(**f32).contiguous()
        self.norm_w = tensors[p + "norm"].to(**f32).contiguous()

    def forward(self, x, step, binding: LayerBinding):
        n = x.shape[0]
        proj = ops.gemm(x, self.w_in)
        out = torch.empty((n, self.nv), dtype=x.dtype, device=x.device)
        ops.forget_gate_recurrence(proj[:, :self.nq + self.nv], proj[:, self.f_at:self.f_at + self.nq], self.lower,
                                   self.f_bias, self.norm_w, self.eps, binding.state, out, step.row_slot, step.row_last,
                                   self.num_heads, self.k_dim, self.v_dim, requests=len(step.segments),
                                   segments=step.plan(segment_plan.planner()))
        return ops.gemm(out, self.w_o)


register_part("mixer", "forget_gate_recurrence", ForgetGateRecurrence)
