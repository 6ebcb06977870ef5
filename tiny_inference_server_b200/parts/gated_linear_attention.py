"""Gated linear attention: a recurrent mixer with a matrix state and a decay per head and key channel."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops, segment_plan
from ..registry import register_part
from .base import BuildContext, LayerBinding, Mixer, StateSpec, WeightSpec
from .window_attention import pad8


class GatedLinearAttention(Mixer):
    """Per head a state ``S`` (``k_dim x v_dim``, float32, zero at the start of a sequence):

    * ``q = Wq h * k_dim ** -0.5``, ``k = Wk h`` (``num_heads`` heads of ``k_dim``), ``v = Wv h`` (heads of ``v_dim``);
    * a decay per head and key channel from a low-rank projection, ``alpha = sigmoid(Wa2 (Wa1 h) + a2.b) ** (1 / tau)``;
    * ``S <- diag(alpha) S + k v^T;  o = S^T q`` (the decay acts on the rows of S, one per key channel; o is read from
      the updated S);
    * every head's ``o`` is divided by its root mean square over ``v_dim`` (``eps`` inside the root) and multiplied by
      ``norm`` (``v_dim`` weights shared by the heads); the heads side by side times ``gate_act(Wg h)``; then ``Wo``.

    Tensor names below the prefix: ``q, k, v, g, o, a1, a2`` (stored (out, in)), ``a2.b``, ``norm``.  The decay (as
    ``exp(-softplus(-z) / tau)``), the state, the recurrence and the norm are 32-bit; the state lives in the cache
    manager's state slots."""

    graph_safe = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, k_dim: int, v_dim: int, tau: float, decay_rank: int, eps: float,
                 gate_act: str = "silu", prefix: str = ""):
        super().__init__(prefix)
        if not tau > 0:
            raise ValueError(f"tau must be positive, got {tau}")
        if gate_act not in ops.GATE_ACTS:
            raise ValueError(f"gate activation {gate_act!r}: one of {sorted(ops.GATE_ACTS)}")
        self.width, self.num_heads, self.k_dim, self.v_dim = width, num_heads, k_dim, v_dim
        self.tau, self.decay_rank, self.eps, self.gate_act = float(tau), decay_rank, float(eps), gate_act
        self.nq = num_heads * k_dim
        self.nv = num_heads * v_dim
        # columns of the fused input projection: q | k | v | gate | a1, each block on a multiple of 8
        self.gate_at = pad8(2 * self.nq + self.nv)
        self.low_at = self.gate_at + pad8(self.nv)
        self.cols = self.low_at + pad8(decay_rank)
        self.w_in = self.w_low = self.w_o = self.a_bias = self.power = self.norm_w = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None):
        m = cfg.layers[layer_index]["mixer"]
        if "decay_rank" not in m:
            raise ValueError(f"layers[{layer_index}].mixer: the rank of the decay's projection is not known "
                             f"(read the configuration with registry.config_from_folder)")
        return cls(cfg.hidden_size, m["heads"], m["dim"], m["vdim"], m["tau"], m["decay_rank"], cfg.rms_norm_eps,
                   prefix=prefix)

    def step_planners(self):
        return (segment_plan.planner(),)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads * self.k_dim * self.v_dim,), torch.float32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nq, self.width)),
                "v": WeightSpec((self.nv, self.width)), "g": WeightSpec((self.nv, self.width)),
                "a1": WeightSpec((self.decay_rank, self.width)), "a2": WeightSpec((self.nq, self.decay_rank)),
                "a2.b": WeightSpec((self.nq,), init="uniform", lo=0.0, hi=4.0),
                "norm": WeightSpec((self.v_dim,), init="ones_normal"), "o": WeightSpec((self.width, self.nv))}

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        at = 0
        for name, n in (("q", self.nq), ("k", self.nq), ("v", self.nv)):
            w[:, at:at + n] = tensors[p + name].to(ctx.dtype).t()
            at += n
        w[:, self.gate_at:self.gate_at + self.nv] = tensors[p + "g"].to(ctx.dtype).t()
        w[:, self.low_at:self.low_at + self.decay_rank] = tensors[p + "a1"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        low = torch.zeros((pad8(self.decay_rank), pad8(self.nq)), dtype=ctx.dtype)
        low[:self.decay_rank, :self.nq] = tensors[p + "a2"].to(ctx.dtype).t()
        self.w_low = low.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.a_bias = tensors[p + "a2.b"].to(**f32).contiguous()
        self.norm_w = tensors[p + "norm"].to(**f32).contiguous()
        self.power = torch.full((self.num_heads,), 1.0 / self.tau, dtype=torch.float64).to(**f32)

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        proj = ops.gemm(x, self.w_in)
        low = ops.gemm(proj[:, self.low_at:], self.w_low)
        out = torch.empty((n, self.nv), dtype=x.dtype, device=x.device)
        ops.gated_linear_attention(proj[:, :2 * self.nq + self.nv], low[:, :self.nq], self.power, self.a_bias,
                                   proj[:, self.gate_at:self.gate_at + self.nv], self.norm_w, self.eps, self.k_dim ** -0.5,
                                   binding.state, out, step.row_slot, step.row_last, self.num_heads, self.k_dim, self.v_dim,
                                   requests=len(step.segments), segments=step.plan(segment_plan.planner()),
                                   gate_act=self.gate_act)
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
