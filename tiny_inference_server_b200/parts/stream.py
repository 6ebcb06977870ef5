"""The residual stream of a step: a float32 tensor (rows, width) and at most one update
that has not been added yet.  The pending update is added by the norm that reads the
stream next (one fused kernel), which is where every pre-norm block wants it.

A part whose last product can add to the stream itself is given a *sink* instead (``sink``); what it
hands back is the next norm's output short of one factor per row (``kernels.ops.ScaledRows``), kept
here until that norm asks for it.

A layer whose two sublayers read the same stream hands in two updates (``add(first)``, ``add(second, also=True)``): both
stay pending, and a norm that can add two (``add_norm(..., delta_b=)``) adds them in the kernel that normalises the sum;
``normed_pair`` gives the outputs of two norms of that sum from one kernel where the first norm can (``add_norm_pair``).

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
        self.pending_b: Optional[torch.Tensor] = None     # a second update beside the first (no norm of its own)
        self.ready: Optional[ops.ScaledRows] = None

    def sink(self, norm, dtype: torch.dtype):
        """A sink for the part that runs before ``norm``, or None when this step's rows or the norm do
        not allow one.  ``dtype``: the compute dtype of the products."""
        if self.pending is not None or not ops.sink_usable(self.values, dtype):
            return None
        return norm.sink(self.values)

    def _settle(self) -> None:
        """Add the pending update now, without a norm of the sum."""
        if self.pending_b is not None:
            ops.residual_add(self.values, self.pending_b)
            self.pending_b = None
        if self.pending is None:
            return
        if self.pending_post is not None:
            ops.add_rmsnorm(self.values, self.pending, None, 0.0, None, delta_norm=self.pending_post.as_delta_norm())
        else:
            ops.residual_add(self.values, self.pending)
        self.pending = self.pending_post = None

    def add(self, update, post=None, also: bool = False) -> None:
        """``update``: a part's result, or the ``ScaledRows`` of a part that has added its result itself.
        ``post``: a norm (with ``as_delta_norm``) that the update passes before it is added.  ``also``: the update
        joins the one that is pending (both were made from the same stream) instead of settling it."""
        if also and post is None and not isinstance(update, ops.ScaledRows) and self.pending is not None \
                and self.pending_post is None and self.pending_b is None:
            self.pending_b = update
            return
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
        if self.pending_b is not None and (self.pending_post is not None or not hasattr(norm, "add_norm_pair")):
            ops.residual_add(self.values, self.pending_b)
            self.pending_b = None
        delta, self.pending = self.pending, None
        post, self.pending_post = self.pending_post, None
        delta_b, self.pending_b = self.pending_b, None
        if post is not None:
            return norm.add_norm(self.values, delta, delta_norm=post.as_delta_norm())
        if delta_b is not None:
            return norm.add_norm(self.values, delta, delta_b=delta_b)
        return norm.add_norm(self.values, delta)

    def normed_pair(self, norm_a, norm_b):
        """(norm_a(sum), norm_b(sum)) with sum = values + everything pending, which stays in ``values``: one kernel where
        ``norm_a`` has ``add_norm_pair``, else one norm after the other."""
        if self.ready is None and self.pending_post is None and hasattr(norm_a, "add_norm_pair"):
            delta, self.pending = self.pending, None
            delta_b, self.pending_b = self.pending_b, None
            return norm_a.add_norm_pair(self.values, delta, delta_b, norm_b)
        a = self.normed(norm_a)
        return a, norm_b.forward(self.values)

    def flush(self) -> torch.Tensor:
        self.ready = None
        self._settle()
        return self.values
