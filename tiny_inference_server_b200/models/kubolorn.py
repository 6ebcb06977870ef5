"""The Kubolorn decoder, put together from parts: a scaled embedding plus a row of a second table addressed by a hash of
the token and its predecessor, under a norm of its own; layers whose two sublayers read the same stream, ``x +=
mixer(norm1(x)) + ff(norm2(x))``, each sublayer behind a short causal convolution of its input (``h + conv(h)``); the mixer
is gated linear attention, or attention whose values are its keys beside a selective state space; the feed-forward is two
matrices around an activation or a routed mixture of such; every norm is an RMS norm in groups; a span of layers runs
several times in a row with the same weights, each pass with cache and state of its own; logits from the embedding matrix.

Tensor names::

    embed                        (vocab, width)
    bigram                       (buckets + 1, width)     the last row is a sequence's first token's
    embed.norm                   (width,)
    l<i>.norm1, l<i>.norm2       (width,)
    l<i>.canon1, l<i>.canon2     (width, taps)            the convolutions in front of the mixer and the feed-forward
    l<i>.mix.*                   the mixer's tensors (``parts.gated_linear_attention.GatedLinearAttention``; or, below
                                 ``left.`` and ``right.``, ``parts.sink_attention.TiedValueAttention`` and
                                 ``parts.state_space.SelectiveStateSpace``)
    l<i>.mlp.*                   the feed-forward's tensors (``parts.feed_forward.ActMLP``, ``RoutedExperts``)
    final.norm                   (width,)

Linear weights are stored ``(out, in)``.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.model_config import KubolornConfig
from ..parts.base import BuildContext, StateSpec
from ..parts.block import Block
from ..parts.embedding import Embedding, LMHead, PairHashEmbedding
from ..parts.feed_forward import ActMLP, RoutedExperts
from ..parts.gated_linear_attention import GatedLinearAttention
from ..parts.norms import RMSNormGrouped
from ..parts.short_conv import CausalConv
from ..parts.side_by_side import SideBySide
from ..parts.sink_attention import TiedValueAttention
from ..parts.state_space import SelectiveStateSpace
from ..parts.stream import ResidualStream
from ..registry import register_architecture
from .base import Model, ScheduleEntry, StepOutput

#: the activations that the design fixes
DENSE_ACT = "gelu_tanh"
EXPERT_ACT = "relu2"


def _mixer(cfg: KubolornConfig, i: int, prefix: str):
    layer = cfg.layers[i]
    if layer["type"] == "gla":
        return GatedLinearAttention.from_config(cfg, prefix=prefix, layer_index=i)
    m = layer["mixer"]
    left = TiedValueAttention.from_config(cfg, prefix=prefix + "left.", layer_index=i, mixer=m["left"])
    right = SelectiveStateSpace.from_config(cfg, prefix=prefix + "right.", layer_index=i, mixer=m["right"])
    return SideBySide(left, right, m.get("left_scale", 1.0), m.get("right_scale", 1.0), prefix=prefix)


def _feed_forward(cfg: KubolornConfig, i: int, prefix: str):
    f = cfg.layers[i].get("mlp")
    if f is None:
        return None
    if f["kind"] == "dense":
        return ActMLP(cfg.hidden_size, f["ff"], DENSE_ACT, prefix=prefix)
    # the largest logits choose, the softmax over the chosen logits weighs; experts without a gate
    return RoutedExperts.from_config(cfg, prefix=prefix, layer_index=i, scores="softmax_chosen", correction=False,
                                     unit_act=EXPERT_ACT)


class KubolornModel(Model):
    def __init__(self, cfg: KubolornConfig):
        super().__init__()
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.max_positions = cfg.max_context
        width, eps, groups = cfg.hidden_size, cfg.rms_norm_eps, cfg.norm_groups

        def norm(name):
            return RMSNormGrouped(width, groups, eps, prefix=name, weight_name="")

        def canon(prefix, name):
            if cfg.canon_taps is None:
                return None
            return CausalConv([width], cfg.canon_taps, [name], prefix=prefix, residual=True)

        if cfg.bigram is not None:
            b = cfg.bigram
            self.embedding = PairHashEmbedding(cfg.vocab_size, width, b["buckets"], b["mul_prev"], b["mul_cur"],
                                               weight_name="embed", pairs_name="bigram", scale=cfg.embedding_scale)
        else:
            self.embedding = Embedding(cfg.vocab_size, width, weight_name="embed", scale=cfg.embedding_scale)
        self.embed_norm = norm("embed.norm")
        self.blocks: List[Block] = []
        for i in range(cfg.num_layers):
            p = f"l{i}."
            ffn = _feed_forward(cfg, i, p + "mlp.")
            self.blocks.append(Block(norm(p + "norm1"), _mixer(cfg, i, p + "mix."), norm(p + "norm2") if ffn is not None else None,
                                     ffn, prefix=p, input_filter=canon(p, "canon1"), parallel=True,
                                     ffn_filter=canon(p, "canon2") if ffn is not None else None))
        self.final_norm = norm("final.norm")
        self.lm_head = LMHead(cfg.vocab_size, width, self.embedding)
        # a layer of the looped span appears once per pass: one block, a cache plane and a state per entry
        self.entries = [ScheduleEntry(self.blocks[i]) for i in cfg.layer_runs()]
        self._prev = None

    def top_parts(self):
        return [self.embedding, self.embed_norm, *self.blocks, self.final_norm, self.lm_head]

    def extra_states(self, ctx: BuildContext) -> Dict[str, StateSpec]:
        if isinstance(self.embedding, PairHashEmbedding):
            return {"previous_token": self.embedding.state_spec()}
        return {}

    def bind(self, cache) -> None:
        super().bind(cache)
        self._prev = cache.states.get("previous_token")

    def forward(self, step, want_rows, aux: bool = False) -> StepOutput:
        if self._prev is not None:
            x = self.embedding.forward(step.tokens, step, self._prev)
        else:
            x = self.embedding.forward(step.tokens)
        # the stream starts as the normed embedding, in 32-bit
        stream = ResidualStream(self.embed_norm.in_place(x))
        for e in self.entries:
            e.block.forward(stream, step, e.binding)
        h = stream.normed(self.final_norm)
        if not getattr(step, "want_identity", False):
            h = h.index_select(0, want_rows)
        return StepOutput(main=self.lm_head.forward(h))


def build(cfg: KubolornConfig) -> KubolornModel:
    return KubolornModel(cfg)


register_architecture(KubolornConfig.architecture, KubolornConfig, build)
