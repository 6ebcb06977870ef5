"""Attention whose keys and values are expanded from one compressed vector per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, window_plan
from ..registry import register_part
from .base import BuildContext, KVSpec, LayerBinding, Mixer, WeightSpec
from .positions import RotaryRescaled
from .window_attention import pad8


class LatentAttention(Mixer):
    """Causal softmax attention over a cache that holds, per token, a latent vector ``c`` (``rank`` elements) and
    one rotated key slice (``rot_dim`` elements) shared by all heads:

    * ``q = Wq h``: per head ``flat_dim`` elements that meet an unrotated key and ``rot_dim`` that are rotated;
    * ``Wdkv h``: the first ``rank`` elements, divided by their root mean square (``eps`` inside the root) and
      multiplied by ``dkv.norm``, are ``c``; the last ``rot_dim``, rotated, are the shared key slice;
    * head h: key ``Wuk[h] c``, value ``Wuv[h] c``; score ``(q_flat . Wuk[h] c + q_rot . k_rot) * scale``;
      the rotation (``position``, a ``RotaryHalf`` family member over the first ``position.rotary_dim`` of the
      ``rot_dim`` channels) is applied to ``q_rot`` and the key slice only;
    * softmax over the keys ``0..p`` (``window`` W: over ``p-W+1..p``, and the cache gives older pages back) with,
      when ``has_sink``, one more term ``exp(sink[h])`` in the denominator that has no key and no value;
    * ``head_gate``: head h's output times ``sigmoid(Wg h)_h``, one number per head, from the same input;
    * ``Wo`` on the heads' outputs side by side.

    ``rot_dim`` 0 (``position`` None): there is no rotated slice; queries, keys and the cache rows hold nothing of it.

    The products with ``Wuk`` and ``Wuv`` are taken out of the loop over keys: ``q_flat . Wuk[h] c = (Wuk[h]^T
    q_flat) . c``, and ``sum_j p_j Wuv[h] c_j = Wuv[h] (sum_j p_j c_j)``.  So the attention kernel sees one kv head
    whose key rows are ``[c | k_rot]`` and whose value rows are the first ``rank`` elements of the same rows, and
    queries ``[Wuk[h]^T q_flat | q_rot]``; the cache holds nothing else.

    Tensor names below the prefix: ``q, dkv, uk, uv, o, g`` (stored (out, in)), ``dkv.norm``, ``sink``."""

    graph_safe = True
    fuses_residual = True

    def __init__(self, width: int, num_heads: int, flat_dim: int, rot_dim: int, v_dim: int, rank: int, scale: float,
                 eps: float, position: Optional[RotaryRescaled], has_sink: bool = True, window: Optional[int] = None,
                 head_gate: bool = False, prefix: str = ""):
        super().__init__(prefix)
        if (rot_dim > 0) != (position is not None):
            raise ValueError("a rotated slice needs a position encoding, and only a rotated slice does")
        self.window, self.head_gate = window, head_gate
        self.width, self.num_heads, self.flat_dim, self.rot_dim = width, num_heads, flat_dim, rot_dim
        self.v_dim, self.rank, self.scale, self.eps = v_dim, rank, float(scale), float(eps)
        self.position, self.has_sink = position, has_sink
        self.q_dim = flat_dim + rot_dim                  # a head's share of the query projection
        self.row = rank + rot_dim                        # a cache row, and a head's query as the kernel sees it
        self.nq = num_heads * self.q_dim
        self.dkv_at = pad8(self.nq)
        self.gate_at = self.dkv_at + pad8(self.row)          # the per-head gates, behind the compressed projection
        self.cols = self.gate_at + (pad8(num_heads) if head_gate else 0)
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.c_weight = self.sink = None

    @classmethod
    def from_config(cls, cfg, prefix: str, layer_index: int, lag: int = 0, position=None, has_sink: bool = True,
                    head_gate: bool = False):
        m = cfg.layers[layer_index]["mixer"]
        rot_dim = m.get("rot_dim", 0)
        pos = None
        if rot_dim:
            rot = m["rot"]
            pos = RotaryRescaled(rot_dim, rot["base"], cfg.max_context, scaling=rot.get("scaling"),
                                 rotary_dim=rot.get("dims", rot_dim))
        mask = m.get("mask")
        return cls(cfg.hidden_size, m["heads"], m["dim"], rot_dim, m["vdim"], m["kv_rank"], m["scale"],
                   cfg.rms_norm_eps, pos, has_sink=has_sink, window=mask["size"] if mask else None,
                   head_gate=head_gate, prefix=prefix)

    def children(self):
        return (self.position,) if self.position is not None else ()

    def kv_spec(self) -> KVSpec:
        # one kv head; the values are a slice of the key rows, so a page holds no value rows of its own
        return KVSpec(1, self.row, self.window, 0, k_dim=self.row, v_dim=0)

    def step_planners(self):
        return (window_plan.planner(self.num_heads),)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"q": WeightSpec((self.nq, self.width)), "dkv": WeightSpec((self.row, self.width)),
                 "dkv.norm": WeightSpec((self.rank,), init="ones_normal"),
                 "uk": WeightSpec((self.num_heads * self.flat_dim, self.rank)),
                 "uv": WeightSpec((self.num_heads * self.v_dim, self.rank)),
                 "o": WeightSpec((self.width, self.num_heads * self.v_dim))}
        if self.has_sink:
            specs["sink"] = WeightSpec((self.num_heads,), init="uniform", lo=-1.0, hi=1.0)
        if self.head_gate:
            specs["g"] = WeightSpec((self.num_heads, self.width))
        return specs

    def load(self, tensors, ctx: BuildContext) -> None:
        p = self.prefix
        H = self.num_heads
        w = torch.zeros((self.width, self.cols), dtype=ctx.dtype)
        w[:, :self.nq] = tensors[p + "q"].to(ctx.dtype).t()
        w[:, self.dkv_at:self.dkv_at + self.row] = tensors[p + "dkv"].to(ctx.dtype).t()
        if self.head_gate:
            w[:, self.gate_at:self.gate_at + H] = tensors[p + "g"].to(ctx.dtype).t()
        self.w_in = w.to(ctx.device).contiguous()
        dev = dict(device=ctx.device, dtype=ctx.dtype)
        self.w_uk = tensors[p + "uk"].to(**dev).reshape(H, self.flat_dim, self.rank).contiguous()
        self.w_uv = tensors[p + "uv"].to(**dev).reshape(H, self.v_dim, self.rank).transpose(1, 2).contiguous()
        self.w_o = tensors[p + "o"].to(**dev).t().contiguous()
        self.c_weight = tensors[p + "dkv.norm"].to(device=ctx.device, dtype=torch.float32).contiguous()
        if self.has_sink:
            self.sink = tensors[p + "sink"].to(device=ctx.device, dtype=torch.float32).contiguous()

    def forward(self, x, step, binding: LayerBinding, residual=None):
        n, H = x.shape[0], self.num_heads
        g = binding.kv_group
        table, page_size = step.block_tables[g], step.page_sizes[g]
        proj = ops.gemm(x, self.w_in)
        q = torch.empty((n, H * self.row), dtype=x.dtype, device=x.device)
        # c and the rotated key slice into the cache; the rotated query slices into their places of q
        cos, sin = (self.position.cos, self.position.sin) if self.position is not None else (None, None)
        ops.latent_prepare(proj, self.dkv_at, H, self.flat_dim, self.rot_dim, self.rank, self.c_weight, self.eps,
                           cos, sin, q, binding.k_pages, table, step.positions, step.row_slot, page_size, step.fault)
        ops.gemm_heads(proj[:, :self.nq].unflatten(1, (H, self.q_dim))[:, :, :self.flat_dim], self.w_uk,
                       q.unflatten(1, (H, self.row))[:, :, :self.rank])
        latent = torch.empty((n, H * self.rank), dtype=x.dtype, device=x.device)
        # a gate per head is one number for all of the head's elements, so it passes the product with Wuv unchanged
        gate = proj[:, self.gate_at:self.gate_at + H] if self.head_gate else None
        ops.window_attention(q, gate, latent, binding.k_pages, binding.k_pages[..., :self.rank], table, step.positions,
                             step.row_slot, H, page_size, self.window, self.scale, None, None, step.fault, step,
                             sink=self.sink, gate_per_head=self.head_gate)
        heads = torch.empty((n, H * self.v_dim), dtype=x.dtype, device=x.device)
        ops.gemm_heads(latent.unflatten(1, (H, self.rank)), self.w_uv, heads.unflatten(1, (H, self.v_dim)))
        return ops.gemm(heads, self.w_o, sink=residual)


register_part("mixer", "latent_attention", LatentAttention)
