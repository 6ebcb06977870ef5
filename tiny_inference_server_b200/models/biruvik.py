"""The Biruvik decoder, put together from parts: scaled embedding; layers ``x += post(mixer(pre(x)))`` and, where the
layer has one, ``x += post(ff(pre(x)))`` — a norm in front of and behind every sublayer, each with one number as its
weight; the mixer is differential attention, windowed attention over a compressed cache with a gate per head, or a
recurrence whose forget gate also writes; the feed-forward is two matrices around an activation; final norm; logits
from a matrix of their own, bounded by a tanh.

Tensor names::

    embed                                   (vocab, width)
    l<i>.norm1, l<i>.norm1b                 ()  one number each: in front of and behind the mixer
    l<i>.norm2, l<i>.norm2b                 ()  the same around the feed-forward (layers that have one)
    l<i>.mix.*                              the mixer's tensors (``parts.diff_attention.DifferentialAttention``,
                                            ``parts.latent_attention.LatentAttention``,
                                            ``parts.gated_recurrence.ForgetGateRecurrence``)
    l<i>.mlp.up, l<i>.mlp.down              (``parts.feed_forward.ActMLP``)
    final.norm                              ()
    head                                    (vocab, width)

Linear weights are stored ``(out, in)``.
"""
from __future__ import annotations

from typing import List

from ..config.model_config import BiruvikConfig
from ..parts.block import Block
from ..parts.diff_attention import DifferentialAttention
from ..parts.embedding import Embedding, LMHead
from ..parts.feed_forward import ActMLP
from ..parts.gated_recurrence import ForgetGateRecurrence
from ..parts.latent_attention import LatentAttention
from ..parts.norms import RMSNormScalar
from ..parts.stream import ResidualStream
from ..registry import register_architecture
from .base import Model, ScheduleEntry, StepOutput


def _mixer(cfg: BiruvikConfig, i: int, prefix: str):
    kind = cfg.layers[i]["type"]
    if kind == "attention":
        return DifferentialAttention.from_config(cfg, prefix=prefix, layer_index=i)
    if kind == "latent_attention":
        # no rotated slice and no keyless softmax term in this design; one sigmoid gate per head
        return LatentAttention.from_config(cfg, prefix=prefix, layer_index=i, has_sink=False, head_gate=True)
    return ForgetGateRecurrence.from_config(cfg, prefix=prefix, layer_index=i)


class BiruvikModel(Model):
    def __init__(self, cfg: BiruvikConfig):
        super().__init__()
        self.config = cfg
        self.vocab_size = cfg.vocab_size
        self.max_positions = cfg.max_context
        width, eps = cfg.hidden_size, cfg.rms_norm_eps

        def norm(name):
            return RMSNormScalar(width, eps, prefix=name, weight_name="")

        self.embedding = Embedding(cfg.vocab_size, width, weight_name="embed", scale=cfg.embedding_scale)
        self.blocks: List[Block] = []
        for i, layer in enumerate(cfg.layers):
            p = f"l{i}."
            has_ff = layer.get("mlp") is not None
            self.blocks.append(Block(
                norm(p + "norm1"), _mixer(cfg, i, p + "mix."),
                norm(p + "norm2") if has_ff else None,
                ActMLP.from_config(cfg, prefix=p + "mlp.", layer_index=i) if has_ff else None,
                prefix=p, post_mixer_norm=norm(p + "norm1b"), post_ffn_norm=norm(p + "norm2b") if has_ff else None))
        self.final_norm = norm("final.norm")
        self.lm_head = LMHead(cfg.vocab_size, width, None, weight_name="head", softcap=cfg.logit_softcap)
        self.entries = [ScheduleEntry(b) for b in self.blocks]

    def top_parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.lm_head]

    def forward(self, step, want_rows, aux: bool = False) -> StepOutput:
        stream = ResidualStream(self.embedding.forward(step.tokens))
        for e in self.entries:
            e.block.forward(stream, step, e.binding)
        h = stream.normed(self.final_norm)
        if not getattr(step, "want_identity", False):
            h = h.index_select(0, want_rows)
        return StepOutput(main=self.lm_head.forward(h))


def build(cfg: BiruvikConfig) -> BiruvikModel:
    return BiruvikModel(cfg)


register_architecture(BiruvikConfig.architecture, BiruvikConfig, build)
