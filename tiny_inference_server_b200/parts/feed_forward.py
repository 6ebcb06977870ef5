"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import BuildContext, FeedForward, WeightSpec


class SwiGLU(FeedForward):
    """``(silu(x W1) * (x W2)) W3`` (upstream ``swiglu`` and ``ffn_router``,
    main_models_new.py:44-60); weights ``(in, out)``: W1 gate and W2 up ``(width, hidden)``,
    W3 ``(hidden, width)``.  On the device gate and up are one matrix ``(width, 2*hidden)``
    whose columns alternate in blocks of 32 gates and 32 ups (when 32 divides the hidden size;
    else all gates, then all ups), so that one 64-column strip of the product holds both
    factors of 32 outputs and the gating can be the product's epilogue."""

    accepts_scaled_rows = True
    fuses_residual = True

    def __init__(self, width: int, hidden: int, prefix: str = "", names: Optional[Dict[str, str]] = None,
                 stored_out_in: bool = False):
        super().__init__(prefix)
        self.width = width
        self.hidden = hidden
        self.stored_out_in = stored_out_in        # the three matrices are stored (out, in) instead of (in, out)
        self.names = {"gate": "swig.linear1.weight", "up": "swig.linear2.weight", "down": "fc.weight"}
        if names:
            self.names.update(names)
        self.w_gate_up = None
        self.w_down = None
        self.block = hidden

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        return cls(cfg.hidden_size, cfg.ffn_hidden, prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        wide, tall = (self.width, self.hidden), (self.hidden, self.width)
        if self.stored_out_in:
            wide, tall = tall, wide
        return {self.names["gate"]: WeightSpec(wide), self.names["up"]: WeightSpec(wide),
                self.names["down"]: WeightSpec(tall)}

    def load(self, tensors, ctx: BuildContext) -> None:
        gate = tensors[self.prefix + self.names["gate"]]
        up = tensors[self.prefix + self.names["up"]]
        down = tensors[self.prefix + self.names["down"]]
        if self.stored_out_in:
            gate, up, down = gate.t(), up.t(), down.t()
        self.block = 32 if self.hidden % 32 == 0 else self.hidden
        nb = self.hidden // self.block
        both = torch.stack([gate.reshape(self.width, nb, self.block), up.reshape(self.width, nb, self.block)], dim=2)
        self.w_gate_up = both.reshape(self.width, 2 * self.hidden).to(device=ctx.device, dtype=ctx.dtype).contiguous()
        self.w_down = down.to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, x, step=None, residual=None):
        h = ops.gemm_swiglu(x, self.w_gate_up, self.hidden, self.block)
        return ops.gemm(h, self.w_down, sink=residual)


class ClampedGLU(FeedForward):
    """``g = min(W_gate h + b, limit)``, ``u = clamp(W_up h + b, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + shift)``, output ``W_down y + b``.  Weights stored ``(out, in)``,
    names ``gate, up, down`` with biases ``gate.b, up.b, down.b``.  On the device gate and up are one matrix;
    the bias of the down projection is one more row of its matrix, met by a column of ones that the gating
    kernel writes, so that the product adds it."""

    accepts_scaled_rows = True

    def __init__(self, width: int, hidden: int, limit: float, alpha: float = 1.702, shift: float = 1.0,
                 prefix: str = ""):
        super().__init__(prefix)
        self.width, self.hidden = width, hidden
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.padded = (hidden + 1 + 7) // 8 * 8
        self.w_gate_up = self.w_down = self.b_gate = self.b_up = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        f = cfg.layers[layer_index]["mlp"]
        return cls(cfg.hidden_size, f["ff"], f.get("limit", 0.0), prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "gate": WeightSpec((self.hidden, self.width)), "gate.b": WeightSpec((self.hidden,)),
            "up": WeightSpec((self.hidden, self.width)), "up.b": WeightSpec((self.hidden,)),
            "down": WeightSpec((self.width, self.hidden)), "down.b": WeightSpec((self.width,)),
        }

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        gu = torch.cat([tensors[p + "gate"], tensors[p + "up"]], dim=0).to(ctx.dtype).t()
        self.w_gate_up = gu.to(ctx.device).contiguous()
        down = torch.zeros((self.padded, self.width), dtype=ctx.dtype)
        down[:self.hidden] = tensors[p + "down"].to(ctx.dtype).t()
        down[self.hidden] = tensors[p + "down.b"].to(ctx.dtype)
        self.w_down = down.to(ctx.device).contiguous()
        self.b_gate = tensors[p + "gate.b"].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.b_up = tensors[p + "up.b"].to(device=ctx.device, dtype=torch.float32).contiguous()

    def forward(self, x, step=None):
        gu = ops.gemm(x, self.w_gate_up)
        y = torch.empty((gu.shape[0], self.padded), dtype=gu.dtype, device=gu.device)
        ops.glu_clamped(gu, self.b_gate, self.b_up, self.limit, self.alpha, self.shift, y, self.hidden)
        return ops.gemm(y, self.w_down)


class ActMLP(FeedForward):
    """``W_down act(W_up h)``: two matrices and an activation, no gate, no biases.  ``act``: ``relu2`` (the square of
    relu), ``gelu_tanh`` or ``silu`` (``kernels.ops.ACTIVATIONS``).  Weights stored ``(out, in)``, names ``up, down``."""

    def __init__(self, width: int, hidden: int, act: str = "relu2", prefix: str = ""):
        super().__init__(prefix)
        if act not in ops.ACTIVATIONS:
            raise ValueError(f"activation {act!r}: known are {sorted(ops.ACTIVATIONS)}")
        self.width, self.hidden, self.act = width, hidden, act
        self.w_up = self.w_down = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int):
        f = cfg.layers[layer_index]["mlp"]
        return cls(cfg.hidden_size, f["ff"], f.get("act", "relu2"), prefix=prefix)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"up": WeightSpec((self.hidden, self.width)), "down": WeightSpec((self.width, self.hidden))}

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        self.w_up = tensors[p + "up"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        self.w_down = tensors[p + "down"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()

    def forward(self, x, step=None):
        return ops.gemm(ops.gemm_act(x, self.w_up, self.act), self.w_down)


class RoutedExperts(FeedForward):
    """A mixture of ``experts`` small gated units ``W_down (silu(W_gate h) * (W_up h))`` (no biases), of which every
    token uses ``top``:

    * router: ``z = W_router h`` and ``s = sigmoid(z)`` in 32-bit; an expert is *chosen* by ``s + correction`` and
      *weighted* by ``s``;
    * ``groups`` > 0: the experts form that many equal groups of neighbours; a group's strength is the sum of its
      two largest choosing scores, and only the experts of the ``keep`` strongest groups can be chosen;
    * the ``top`` experts with the largest choosing scores are taken (the lower index on a tie); their weights are
      their ``s`` divided by the sum of those (+ ``weight_eps``);
    * ``shared_hidden`` > 0: one more unit of that hidden size runs for every token and is added times
      ``sigmoid(w_sg . h)``, one number per token.

    Options: ``scores`` ``"softmax_chosen"``: the logits ``z`` themselves choose (the ``top`` largest) and the weights are
    the softmax over the chosen logits only; ``correction`` False: there is no correction tensor; ``unit_act`` (a name of
    ``kernels.ops.ACTIVATIONS``): the experts have no gate, ``W_down act(W_up h)``, and no ``e<i>.gate`` tensors.

    Tensor names below the prefix: ``e<i>.gate, e<i>.up, e<i>.down``, ``router``, ``correction``, ``shared.gate,
    shared.up, shared.down, shared.sg`` (matrices stored (out, in)).  On the device the experts' matrices are stacked:
    gate and up ``(experts, 2, hidden, width)``, down ``(experts, width, hidden)``; the kernels find an expert's rows
    from the token's choice, so nothing is sorted or gathered on the host."""

    WEIGHT_EPS = 1e-20

    def __init__(self, width: int, hidden: int, experts: int, top: int, groups: int = 0, keep: int = 0,
                 shared_hidden: int = 0, prefix: str = "", scores: str = "sigmoid", correction: bool = True,
                 unit_act: Optional[str] = None):
        super().__init__(prefix)
        if scores not in ops.ROUTER_SCORES:
            raise ValueError(f"router scores {scores!r}: known are {sorted(ops.ROUTER_SCORES)}")
        if unit_act is not None and unit_act not in ops.ACTIVATIONS:
            raise ValueError(f"activation {unit_act!r}: known are {sorted(ops.ACTIVATIONS)}")
        self.scores, self.has_correction, self.unit_act = scores, correction, unit_act
        if groups and (experts % groups or not (0 < keep <= groups)):
            raise ValueError(f"{experts} experts in {groups} groups, {keep} kept")
        if top > (experts // groups * keep if groups else experts):
            raise ValueError(f"top {top} exceeds the experts that can be chosen")
        self.width, self.hidden, self.experts, self.top = width, hidden, experts, top
        self.groups, self.keep, self.shared_hidden = groups, keep, shared_hidden
        self.shared = SwiGLU(width, shared_hidden, prefix=prefix + "shared.", stored_out_in=True,
                             names={"gate": "gate", "up": "up", "down": "down"}) if shared_hidden else None
        self.w_gate_up = self.w_down = self.w_router = self.correction = self.w_shared_gate = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, **options):
        f = cfg.layers[layer_index]["mlp"]
        r = f["router"]
        g = r.get("groups") or {}
        s = f.get("shared") or {}
        return cls(cfg.hidden_size, f["expert"]["ff"], r["experts"], r["top"], g.get("count", 0), g.get("keep", 0),
                   s.get("ff", 0), prefix=prefix, **options)

    def children(self):
        return (self.shared,) if self.shared is not None else ()

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"router": WeightSpec((self.experts, self.width))}
        if self.has_correction:
            specs["correction"] = WeightSpec((self.experts,))
        for e in range(self.experts):
            if self.unit_act is None:
                specs[f"e{e}.gate"] = WeightSpec((self.hidden, self.width))
            specs[f"e{e}.up"] = WeightSpec((self.hidden, self.width))
            specs[f"e{e}.down"] = WeightSpec((self.width, self.hidden))
        if self.shared is not None:
            specs["shared.sg"] = WeightSpec((1, self.width))
        return specs

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        dev = dict(device=ctx.device, dtype=ctx.dtype)
        f32 = dict(device=ctx.device, dtype=torch.float32)
        if self.unit_act is None:
            gu = torch.stack([torch.stack([tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"]]) for e in range(self.experts)])
        else:                                   # units without a gate: (experts, hidden, width)
            gu = torch.stack([tensors[f"{p}e{e}.up"] for e in range(self.experts)])
        self.w_gate_up = gu.to(**dev).contiguous()
        self.w_down = torch.stack([tensors[f"{p}e{e}.down"] for e in range(self.experts)]).to(**dev).contiguous()
        self.w_router = tensors[p + "router"].to(**f32).contiguous()
        self.correction = tensors[p + "correction"].to(**f32).contiguous() if self.has_correction else None
        if self.shared is not None:
            self.w_shared_gate = tensors[p + "shared.sg"].to(**f32).reshape(-1).contiguous()

    def forward(self, x, step=None):
        chosen, weights, shared_gate = ops.moe_route(x, self.w_router, self.correction, self.w_shared_gate, self.groups,
                                                     self.keep, self.top, self.WEIGHT_EPS, scores=self.scores)
        shared = self.shared.forward(x, step) if self.shared is not None else None
        return ops.moe_experts(x, chosen, weights, self.w_gate_up, self.w_down, shared, shared_gate, act=self.unit_act)


register_part("ffn", "swiglu", SwiGLU)
register_part("ffn", "routed_experts", RoutedExperts)
register_part("ffn", "clamped_glu", ClampedGLU)
register_part("ffn", "act_mlp", ActMLP)
