"""Token embedding and the output projection onto the vocabulary."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import BuildContext, Part, StateSpec, WeightSpec


class Embedding(Part):
    """``x = E[token] * scale`` (upstream has no scaling: main_models_new.py:177-178,199).  The gathered
    rows start the float32 residual stream; the product with ``scale`` is made there, in 32-bit."""

    def __init__(self, vocab: int, width: int, prefix: str = "", weight_name: str = "embedding.weight",
                 scale: float = 1.0):
        super().__init__(prefix)
        self.scale = float(scale)
        self.vocab = vocab
        self.width = width
        self.weight_name = weight_name
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.vocab, self.width))}

    def load(self, tensors, ctx: BuildContext) -> None:
        self.table = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        out = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        return ops.embed_rows(self.table, tokens, out, self.scale)


class PairHashEmbedding(Embedding):
    """``x = E[token] * scale + P[(previous * mul_prev + token * mul_cur) mod buckets]``: beside the token's own row a row
    of a second table ``P (buckets + 1, width)`` addressed by a hash of the token and the one before it; the first token
    of a sequence has no predecessor and takes the table's last row.  The previous token of a request is per-request
    state (``state_spec``: one int32), which ``forward`` reads for the first row a request has in the step and brings up
    to date."""

    def __init__(self, vocab: int, width: int, buckets: int, mul_prev: int, mul_cur: int, prefix: str = "",
                 weight_name: str = "embedding.weight", pairs_name: str = "bigram", scale: float = 1.0):
        super().__init__(vocab, width, prefix=prefix, weight_name=weight_name, scale=scale)
        if buckets <= 0:
            raise ValueError(f"a hashed table of {buckets} buckets")
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.pairs_name = pairs_name
        self.pairs: Optional[torch.Tensor] = None

    def state_spec(self) -> StateSpec:
        return StateSpec((1,), torch.int32)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = super().weight_specs()
        specs[self.pairs_name] = WeightSpec((self.buckets + 1, self.width))
        return specs

    def load(self, tensors, ctx: BuildContext) -> None:
        super().load(tensors, ctx)
        self.pairs = tensors[self.prefix + self.pairs_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()

    def forward(self, tokens: torch.Tensor, step=None, state: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        return ops.embed_pairs(self.table, self.pairs, tokens, step.positions, step.row_slot, step.row_last, state, out,
                               self.scale, self.buckets, self.mul_prev, self.mul_cur)


class LMHead(Part):
    """``logits = h @ E^T`` with the embedding matrix (tied, main_models_new.py:225-226) or
    with a matrix of its own, ``lm_head.weight (vocab, width)``.  Logits are float32; ``logit_scale``
    multiplies them (the embedding's own scale plays no part here); ``softcap`` c (None: none) then bounds them
    smoothly, ``c * tanh(logits / c)``."""

    def __init__(self, vocab: int, width: int, embedding: Optional[Embedding], prefix: str = "",
                 weight_name: str = "lm_head.weight", logit_scale: float = 1.0, softcap: Optional[float] = None):
        super().__init__(prefix)
        self.logit_scale = float(logit_scale)
        self.softcap = float(softcap) if softcap else None
        self.vocab = vocab
        self.width = width
        self.embedding = embedding            # given: tied
        self.weight_name = weight_name
        self.weight_t: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.embedding is not None:
            return {}
        return {self.weight_name: WeightSpec((self.vocab, self.width))}

    def load(self, tensors, ctx: BuildContext) -> None:
        if self.embedding is None:
            w = tensors[self.prefix + self.weight_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()
            self.weight_t = w.t()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        wt = self.weight_t if self.embedding is None else self.embedding.table.t()
        logits = ops.gemm_f32_out(h, wt)
        if self.logit_scale != 1.0:
            ops.scale_f32(logits, self.logit_scale)
        if self.softcap is not None:
            ops.softcap_f32(logits, self.softcap)
        return logits
