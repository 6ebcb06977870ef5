"""Grouped-query attention whose values are its keys before rotation, with a keyless term in the softmax."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, window_plan
from ..registry import register_part
from .base import BuildContext, KVSpec, LayerBinding, Mixer, WeightSpec
from .positions import RotaryRescaled


class TiedValueAttention(Mixer):
    """Causal softmax attention with ``num_heads`` query heads over ``kv_heads`` key heads (query head h reads key head
    ``h // (num_heads / kv_heads)``), all of ``dim`` elements:

    * ``q = Wq h``, ``k = Wk h``; there is no value projection: the values are the keys as they were projected;
    * ``position`` (a ``RotaryHalf`` family member) rotates the first ``position.rotary_dim`` elements of every query and
      key head by the token's position; the values stay unrotated;
    * ``score = (q . k) * scale`` over the keys ``0..p`` (``window`` W: ``p - W + 1..p``), softmax in 32-bit; with
      ``has_sink`` its denominator holds one more term ``exp(sink[h])``, a term without a key or a value behind it;
    * ``Wo`` on the heads' outputs side by side.

    The cache holds, per token and key head, the rotated key as the key row and the unrotated key as the value row.
    Tensor names below the prefix: ``q, k, o`` (stored (out, in)) and ``sink``."""

    graph_safe = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, kv_heads: int, dim: int, scale: float, position: Optional[RotaryRescaled],
                 has_sink: bool = True, window: Optional[int] = None, prefix: str = ""):
        super().__init__(prefix)
        if num_heads % kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {kv_heads} kv heads")
        self.width, self.num_heads, self.kv_heads, self.dim = width, num_heads, kv_heads, dim
        self.scale, self.position, self.has_sink, self.window = float(scale), position, has_sink, window
        self.nq, self.nk = num_heads * dim, kv_heads * dim
        self.w_in = self.w_o = self.sink = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None, mixer: Optional[dict] = None):
        m = mixer if mixer is not None else cfg.layers[layer_index]["mixer"]
        if m.get("vdim", m["dim"]) != m["dim"]:
            raise ValueError(f"values that are the keys have the keys' width ({m['dim']}), not {m['vdim']}")
        rot = m.get("rot")
        pos = None
        if rot:
            pos = RotaryRescaled(m["dim"], rot["base"], cfg.max_context, scaling=rot.get("scaling"),
                                 rotary_dim=rot.get("dims", m["dim"]))
        mask = m.get("mask")
        return cls(cfg.hidden_size, m["heads"], m["kv_heads"], m["dim"], m["scale"], pos,
                   window=mask["size"] if mask else None, prefix=prefix)

    def children(self):
        return (self.position,) if self.position is not None else ()

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.kv_heads, self.dim, self.window, 0, k_dim=self.dim, v_dim=self.dim)

    def step_planners(self):
        return (window_plan.planner(self.num_heads // self.kv_heads),)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nk, self.width)),
                 "o": WeightSpec((self.width, self.nq))}
        if self.has_sink:
            specs["sink"] = WeightSpec((self.num_heads,), init="uniform", lo=-1.0, hi=1.0)
        return specs

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        w = torch.cat([tensors[p + "q"], tensors[p + "k"]], dim=0).to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        if self.has_sink:
            self.sink = tensors[p + "sink"].to(device=ctx.device, dtype=torch.float32).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n = x.shape[0]
        g = binding.kv_group
        table, page_size = step.block_tables[g], step.page_sizes[g]
        proj = ops.gemm(x, self.w_in)
        pos = self.position
        ops.rotate_tie_store(proj, self.num_heads, self.kv_heads, self.dim, pos.rotary_dim if pos is not None else 0,
                             pos.cos if pos is not None else None, pos.sin if pos is not None else None, binding.k_pages,
                             binding.v_pages, table, step.positions, step.row_slot, page_size, step.fault)
        out = torch.empty((n, self.nq), dtype=x.dtype, device=x.device)
        ops.window_attention(proj[:, :self.nq], None, out, binding.k_pages, binding.v_pages, table, step.positions,
                             step.row_slot, self.num_heads, page_size, self.window, self.scale, None, None, step.fault, step,
                             sink=self.sink)
        return ops.gemm(out, self.w_o, sink=residual)


register_part("mixer", "tied_value_attention", TiedValueAttention)
