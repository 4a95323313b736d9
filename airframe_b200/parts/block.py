"""Arrangements of a layer's parts around the float32 residual stream.

``sandwich``: x += post(mixer(pre(x))); x += post(ff(pre(x))) - norms before
and after both halves; a layer whose feed-forward is of the kind ``none`` has
the first half only (reference order
``src/backend/bindless/pipeline/inference.rs:1096-1251``, net effect
x + norm(a) of ``sh_layer_v1.wgsl:834-849,869-884``).
``prenorm``: x += mixer(pre(x)); x += ff(pre(x)); a layer whose feed-forward
is of the kind ``none`` has the first half only.  Each residual sum is one
kernel with the norm that follows it (the feed-forward's, or the next layer's
first).
``postnorm``: x += post(mixer(x)); x += post(ff(x)): the sublayers read the
stream itself and the only norms stand behind them (each on the sublayer's output,
not on the sum); a layer whose feed-forward is of the kind ``none`` has the first
half only.  On the 16-bit path the kernel of a residual sum also writes the new
stream in 16 bits for the sublayer that reads it next.
"""
from __future__ import annotations

from .. import kernels
from ..config.base import PartSpec
from .base import Block, build_part, register_part
from .linear import as_terms


@register_part("block", "sandwich")
class SandwichBlock(Block):
    roles = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")

    def __init__(self, params, ctx, mixer, feed_forward, norms):
        if not feed_forward.present:
            self.roles = ("pre_mixer", "post_mixer")
        super().__init__(params, ctx, mixer, feed_forward, norms)

    def forward(self, x, batch, view, normed=None, next_pre=None):
        """Updates x in place.  ``normed`` may carry pre_mixer(x) made by the
        previous layer's last kernel; ``next_pre`` is the next layer's first
        norm, whose output is then returned (made by this layer's last kernel)."""
        n = self.norms
        dt = self.ctx.compute_dtype
        h = normed if normed is not None else n["pre_mixer"].forward(x, dt)
        a = self.mixer.forward(h, batch, view)
        if not self.feed_forward.present:
            return n["post_mixer"].add_normed(x, a, then=next_pre, out_dtype=dt)
        h = n["post_mixer"].add_normed(x, a, then=n["pre_feed_forward"], out_dtype=dt)
        f = self.feed_forward.forward(h, batch)
        return n["post_feed_forward"].add_normed(x, f, then=next_pre, out_dtype=dt)

    def first_norm(self):
        return self.norms["pre_mixer"]


@register_part("block", "prenorm")
class PreNormBlock(Block):
    roles = ("pre_mixer", "pre_feed_forward")

    def __init__(self, params, ctx, mixer, feed_forward, norms):
        if not feed_forward.present:
            self.roles = ("pre_mixer",)
        super().__init__(params, ctx, mixer, feed_forward, norms)

    def _add(self, x, a, then, dt):
        """x += a; returns then(x) when a norm follows."""
        if then is not None:
            return then.after_add(x, a, dt)
        kernels.add_scaled_rmsnorm(x, as_terms(a))
        return None

    def forward(self, x, batch, view, normed=None, next_pre=None):
        n = self.norms
        dt = self.ctx.compute_dtype
        h = normed if normed is not None else n["pre_mixer"].forward(x, dt)
        a = self.mixer.forward(h, batch, view)
        if not self.feed_forward.present:
            return self._add(x, a, next_pre, dt)
        h = self._add(x, a, n["pre_feed_forward"], dt)
        return self._add(x, self.feed_forward.forward(h, batch), next_pre, dt)

    def first_norm(self):
        return self.norms["pre_mixer"]


@register_part("block", "postnorm")
class PostNormBlock(Block):
    roles = ("post_mixer", "post_feed_forward")

    def __init__(self, params, ctx, mixer, feed_forward, norms):
        if not feed_forward.present:
            self.roles = ("post_mixer",)
        super().__init__(params, ctx, mixer, feed_forward, norms)
        # "the norm in front of a sublayer" is none: the stream as it stands, in the compute dtype
        self.reader = build_part("norm", PartSpec("as_is", {"size": norms["post_mixer"].size}), ctx)

    def forward(self, x, batch, view, normed=None, next_pre=None):
        n = self.norms
        dt = self.ctx.compute_dtype
        h = normed if normed is not None else self.reader.forward(x, dt)
        a = self.mixer.forward(h, batch, view)
        if not self.feed_forward.present:
            return n["post_mixer"].add_normed(x, a, then=next_pre, out_dtype=dt)
        h = n["post_mixer"].add_normed(x, a, then=self.reader, out_dtype=dt)
        f = self.feed_forward.forward(h, batch)
        return n["post_feed_forward"].add_normed(x, f, then=next_pre, out_dtype=dt)

    def first_norm(self):
        return self.reader
