"""Differential attention: every head runs two softmax maps over the same values and subtracts one from the other."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import ops, window_plan
from ..registry import register_part
from .base import BuildContext, KVSpec, LayerBinding, Mixer, WeightSpec
from .window_attention import pad8


class DifferentialAttention(Mixer):
    """Grouped-query causal attention without rotation whose heads each carry two score maps:

    * ``q = Wq h + bq`` (H heads x 2 maps x ``dim``), ``k = Wk h + bk`` (G kv heads x 2 maps x ``dim``), ``v = Wv h + bv``
      (G kv heads x ``v_dim``); query head h reads kv head ``h // (H / G)``;
    * every (head, map) of q and k is divided by its root mean square over ``dim`` (``eps`` inside the root) and
      multiplied by ``q.norm`` / ``k.norm`` (``dim`` weights shared by all heads and maps);
    * ``q_temp`` = (coef, every): q at position p times ``1 + coef * ln(floor((p + 1) / every) + 1)`` (None: not);
    * map m of head h: ``softmax_j(q[h, m] . k[g, m] * scale)`` over the keys ``j <= p`` (``window`` W: ``p - W < j``),
      times the values: ``a_m``;
    * ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, one number for the layer; ``o = a_1 - lambda a_2``,
      divided by its root mean square over ``v_dim`` (no weight), times ``1 - diff``;
    * ``Wo`` on the heads' outputs side by side.

    How it runs: the cache holds, per kv head, the key row ``[map 1 | map 2]`` (``2 dim`` wide) and the value row.
    The two maps of a head become two query heads of the key row's whole width, each zero where the other map's
    part of the key lies, so that one pass of the attention kernel over a key row and a value row serves both maps
    of every head of the group; a small kernel then combines the pairs.  Scores, softmax, lambda, the combination
    and its norm are 32-bit.

    Tensor names below the prefix: ``q, k, v, o`` (stored (out, in)), ``q.b, k.b, v.b``, ``q.norm, k.norm``,
    ``lq1, lk1, lq2, lk2``."""

    graph_safe = True
    MAPS = 2

    def __init__(self, width: int, num_heads: int, kv_heads: int, dim: int, v_dim: int, scale: float, diff: float,
                 eps: float, q_temp=None, window: Optional[int] = None, biases: bool = True, qk_norm: bool = True,
                 prefix: str = ""):
        super().__init__(prefix)
        if num_heads % kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {kv_heads} kv heads")
        self.width, self.num_heads, self.kv_heads, self.dim, self.v_dim = width, num_heads, kv_heads, dim, v_dim
        self.scale, self.diff, self.eps, self.window = float(scale), float(diff), float(eps), window
        self.temp_coef, self.temp_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
        self.biases, self.qk_norm = biases, qk_norm
        m = self.MAPS
        self.nq, self.nk, self.nv = num_heads * m * dim, kv_heads * m * dim, kv_heads * v_dim
        self.key_row = m * dim                              # a cache row of keys, and a query head as the kernel sees it
        self.no = num_heads * v_dim
        self.cols = pad8(self.nq + self.nk + self.nv)
        self.lam = 0.0
        self.w_in = self.w_o = self.bias = self.q_weight = self.k_weight = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None):
        m = cfg.layers[layer_index]["mixer"]
        temp, mask = m.get("q_temp"), m.get("mask")
        return cls(cfg.hidden_size, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m["diff"],
                   cfg.rms_norm_eps, q_temp=(temp["coef"], temp["every"]) if temp else None,
                   window=mask["size"] if mask else None, prefix=prefix)

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.kv_heads, self.key_row, self.window, 0, k_dim=self.key_row, v_dim=self.v_dim)

    def step_planners(self):
        return (window_plan.planner(self.MAPS * self.num_heads // self.kv_heads),)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"q": WeightSpec((self.nq, self.width)), "k": WeightSpec((self.nk, self.width)),
                 "v": WeightSpec((self.nv, self.width)), "o": WeightSpec((self.width, self.no))}
        if self.biases:
            specs.update({"q.b": WeightSpec((self.nq,)), "k.b": WeightSpec((self.nk,)), "v.b": WeightSpec((self.nv,))})
        if self.qk_norm:
            specs.update({"q.norm": WeightSpec((self.dim,), init="ones_normal"),
                          "k.norm": WeightSpec((self.dim,), init="ones_normal")})
        for name in ("lq1", "lk1", "lq2", "lk2"):
            specs[name] = WeightSpec((self.dim,))
        return specs

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        f32 = dict(device=ctx.device, dtype=torch.float32)
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        at = 0
        for name, n in (("q", self.nq), ("k", self.nk), ("v", self.nv)):
            w[:, at:at + n] = tensors[p + name].to(ctx.dtype).t()
            at += n
        self.w_in = w.to(ctx.device).contiguous()
        self.w_o = tensors[p + "o"].to(device=ctx.device, dtype=ctx.dtype).t().contiguous()
        if self.biases:
            self.bias = torch.cat([tensors[p + n].to(torch.float32).reshape(-1) for n in ("q.b", "k.b", "v.b")]).to(**f32).contiguous()
        if self.qk_norm:
            self.q_weight = tensors[p + "q.norm"].to(**f32).contiguous()
            self.k_weight = tensors[p + "k.norm"].to(**f32).contiguous()
        lq1, lk1, lq2, lk2 = (tensors[p + n].to(torch.float64) for n in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff

    def forward(self, x, step, binding: LayerBinding):
        n, H, m = x.shape[0], self.num_heads, self.MAPS
        g = binding.kv_group
        table, page_size = step.block_tables[g], step.page_sizes[g]
        proj = ops.gemm(x, self.w_in)
        q = torch.empty((n, H * m * self.key_row), dtype=x.dtype, device=x.device)
        ops.head_norm_store(proj, H, self.kv_heads, m, self.dim, self.v_dim, self.bias, self.q_weight, self.k_weight,
                            self.eps, self.temp_coef, self.temp_every, q, binding.k_pages, binding.v_pages, table,
                            step.positions, step.row_slot, page_size, step.fault)
        maps = torch.empty((n, H * m * self.v_dim), dtype=x.dtype, device=x.device)
        ops.window_attention(q, None, maps, binding.k_pages, binding.v_pages, table, step.positions, step.row_slot,
                             H * m, page_size, self.window, self.scale, None, None, step.fault, step)
        out = torch.empty((n, self.no), dtype=x.dtype, device=x.device)
        ops.diff_combine(maps, self.lam, self.eps, 1.0 - self.diff, out, H, self.v_dim, step.row_slot)
        return ops.gemm(out, self.w_o)


register_part("mixer", "differential_attention", DifferentialAttention)
