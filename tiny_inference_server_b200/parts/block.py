"""A pre-norm block: norm, mixer, residual; norm, feed-forward, residual
(upstream ``Transformer_block``, main_models_new.py:139-152).  Two options that upstream's block does
not have: an *input filter* between the first norm and the mixer (a part with ``forward(x, step, state)``,
for instance a short convolution over time, with per-request state of its own), no feed-forward
at all (the block is its first sublayer only), and a norm *behind* a sublayer as well (``post_mixer_norm``,
``post_ffn_norm``): ``x += post(sublayer(norm(x)))``, the update normalised in 32-bit on its way into the stream.  ``parallel``: both sublayers
read the same stream, ``x += mixer(norm1(x)) + ff(norm2(x))``; the feed-forward may then have an input filter of its own
(``ffn_filter``), whose state follows the mixer filter's in the block's filter state."""
from __future__ import annotations

from typing import Optional

import torch

from .base import LayerBinding, Part, StateSpec
from .stream import ResidualStream


class Block(Part):
    def __init__(self, norm_mixer, mixer, norm_ffn, ffn, prefix: str = "", input_filter=None, post_mixer_norm=None,
                 post_ffn_norm=None, parallel: bool = False, ffn_filter=None):
        super().__init__(prefix)
        if ffn_filter is not None and not parallel:
            raise ValueError("only a block whose sublayers read the same stream filters the feed-forward's input")
        if parallel and (post_mixer_norm is not None or post_ffn_norm is not None):
            raise ValueError("a block whose sublayers read the same stream has no norms behind them")
        self.parallel = parallel
        self.ffn_filter = ffn_filter
        self.post_mixer_norm = post_mixer_norm
        self.post_ffn_norm = post_ffn_norm
        self.norm_mixer = norm_mixer
        self.mixer = mixer
        self.norm_ffn = norm_ffn
        self.ffn = ffn
        self.input_filter = input_filter

    def children(self):
        return tuple(p for p in (self.norm_mixer, self.input_filter, self.mixer, self.post_mixer_norm, self.norm_ffn,
                                 self.ffn_filter, self.ffn, self.post_ffn_norm) if p is not None)

    def filter_state_spec(self):
        if self.ffn_filter is not None:
            first = self.input_filter.state_floats if self.input_filter is not None else 0
            return StateSpec((max(1, first + self.ffn_filter.state_floats),), torch.float32)
        return self.input_filter.state_spec() if self.input_filter is not None else None

    def _forward_parallel(self, stream: ResidualStream, step, binding: LayerBinding) -> None:
        mixer, ffn = self.mixer, self.ffn
        if ffn is None:
            a = stream.normed(self.norm_mixer)
        else:
            a, f = stream.normed_pair(self.norm_mixer, self.norm_ffn)
        first = 0
        if self.input_filter is not None:
            a = self.input_filter.forward(a, step, binding.filter_state)
            first = self.input_filter.state_floats
        update = mixer.forward(a, step, binding)
        if ffn is None:
            stream.add(update)
            return
        if self.ffn_filter is not None:
            f = self.ffn_filter.forward(f, step, binding.filter_state[:, first:])
        stream.add(update)
        stream.add(ffn.forward(f, step), also=True)

    def forward(self, stream: ResidualStream, step, binding: LayerBinding, following: Optional["Block"] = None) -> None:
        """``following``: the block that reads the stream after this one, if the caller knows it; its first
        norm can then be folded into this block's last product and that block's first one."""
        mixer, ffn = self.mixer, self.ffn
        if self.parallel:
            self._forward_parallel(stream, step, binding)
            return
        if self.post_mixer_norm is not None or self.post_ffn_norm is not None:
            # an update that passes a norm cannot be added by the product that makes it (the norm needs whole rows):
            # the norm behind a sublayer, the sum and the norm in front of the next sublayer are one kernel instead
            a = stream.normed(self.norm_mixer)
            if self.input_filter is not None:
                a = self.input_filter.forward(a, step, binding.filter_state)
            stream.add(mixer.forward(a, step, binding), post=self.post_mixer_norm)
            if ffn is not None:
                stream.add(ffn.forward(stream.normed(self.norm_ffn), step), post=self.post_ffn_norm)
            return
        if self.input_filter is not None or ffn is None:
            # the mixer reads the filter's output, whole rows; the norm before the feed-forward can still be folded
            # into the mixer's last product and the feed-forward's first one
            a = stream.normed(self.norm_mixer)
            if self.input_filter is not None:
                a = self.input_filter.forward(a, step, binding.filter_state)
            if ffn is None:
                stream.add(mixer.forward(a, step, binding))
                return
            if mixer.fuses_residual and ffn.accepts_scaled_rows:
                stream.add(mixer.forward(a, step, binding, residual=stream.sink(self.norm_ffn, a.dtype)))
            else:
                stream.add(mixer.forward(a, step, binding))
            stream.add(ffn.forward(stream.normed(self.norm_ffn, scaled=ffn.accepts_scaled_rows), step))
            return
        a = stream.normed(self.norm_mixer, scaled=mixer.accepts_scaled_rows)
        if mixer.fuses_residual and ffn.accepts_scaled_rows:
            stream.add(mixer.forward(a, step, binding, residual=stream.sink(self.norm_ffn, a.dtype)))
        else:
            stream.add(mixer.forward(a, step, binding))
        f = stream.normed(self.norm_ffn, scaled=ffn.accepts_scaled_rows)
        if ffn.fuses_residual and following is not None and following.mixer.accepts_scaled_rows:
            stream.add(ffn.forward(f, step, residual=stream.sink(following.norm_mixer, f.dtype)))
        else:
            stream.add(ffn.forward(f, step))
