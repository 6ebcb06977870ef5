"""The residual stream of a step: a float32 tensor (rows, width) and at most one update
that has not been added yet.  The pending update is added by the norm that reads the
stream next (one fused kernel), which is where every pre-norm block wants it.

A part whose last product can add to the stream itself is given a *sink* instead (``sink``); what it
hands back is the next norm's output short of one factor per row (``kernels.ops.ScaledRows``), kept
here until that norm asks for it.

An update may also pass a norm of its own on its way into the stream (``add(update, post=norm)``, a block with a norm
behind each sublayer): the same fused kernel normalises the update, adds it and normalises the sum."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class ResidualStream:
    def __init__(self, values: torch.Tensor):
        assert values.dtype == torch.float32
        self.values = values
        self.pending: Optional[torch.Tensor] = None
        self.pending_post = None                  # the norm that the pending update passes before it is added
        self.ready: Optional[ops.ScaledRows] = None

    def sink(self, norm, dtype: torch.dtype):
        """A sink for the part that runs before ``norm``, or None when this step's rows or the norm do
        not allow one.  ``dtype``: the compute dtype of the products."""
        if self.pending is not None or not ops.sink_usable(self.values, dtype):
            return None
        return norm.sink(self.values)

    def _settle(self) -> None:
        """Add the pending update now, without a norm of the sum."""
        if self.pending is None:
            return
        if self.pending_post is not None:
            ops.add_rmsnorm(self.values, self.pending, None, 0.0, None, delta_norm=self.pending_post.as_delta_norm())
        else:
            ops.residual_add(self.values, self.pending)
        self.pending = self.pending_post = None

    def add(self, update, post=None) -> None:
        """``update``: a part's result, or the ``ScaledRows`` of a part that has added its result itself.
        ``post``: a norm (with ``as_delta_norm``) that the update passes before it is added."""
        if isinstance(update, ops.ScaledRows):
            if post is not None:
                raise ValueError("an update that has been added already cannot pass a norm")
            self.ready = update
            return
        self.ready = None
        self._settle()
        self.pending, self.pending_post = update, post

    def normed(self, norm, scaled: bool = False):
        """norm(values + pending); the sum stays in ``values``.  ``scaled``: the reader takes ``ScaledRows``."""
        ready, self.ready = self.ready, None
        if ready is not None:
            if ready.norm is norm:
                return ready if scaled else ready.dense()
            return norm.add_norm(self.values, None)        # made for another norm: the stream itself is whole
        delta, self.pending = self.pending, None
        post, self.pending_post = self.pending_post, None
        if post is not None:
            return norm.add_norm(self.values, delta, delta_norm=post.as_delta_norm())
        return norm.add_norm(self.values, delta)

    def flush(self) -> torch.Tensor:
        self.ready = None
        self._settle()
        return self.values
