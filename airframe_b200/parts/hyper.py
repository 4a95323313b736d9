"""A layer around a residual stream that is kept in several copies (hyper-connections).

The model holds ``streams`` copies x_1 .. x_S of the stream, all equal to the
embedding's output at the start; the model's result is their sum.  A sublayer q
(the mixer, then the feed-forward) reads one weighted sum of them and rewrites
all of them at once:

    u    = sum_s in_q[s] x_s
    y    = scale_q * sublayer(norm_q(u))                (scale_q: a per-channel layer scale, optional)
    x_t <- sum_s mix_q[s, t] x_s + out_q[t] y           (every x_t from the old streams)

With one stream and no connection weights this is the plain pre-norm layer
x += scale * sublayer(norm(x)).  The streams lie side by side in one float32 row
[tokens, streams * width]; every sum is 32-bit.  A rewrite and the read and norm of
the sublayer that follows (the feed-forward's, or the next layer's mixer's) are one kernel.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import WeightDecl
from .base import Block, register_part
from .linear import as_terms
from .norm import RmsNorm


class StreamReader:
    """What a sublayer reads of the streams: norm(sum_s in[s] x_s).  Stands where a block's first norm stands."""
    graph_safe = True

    def __init__(self, block, which: int):
        self.block, self.which = block, which

    @property
    def norm(self):
        return self.block.norms["pre_mixer" if self.which == 0 else "pre_feed_forward"]

    @property
    def in_w(self):
        return self.block.conn[self.which][0]

    def forward(self, x, out_dtype, rows=None):
        if rows is not None:
            raise ConfigError("hyper: a sublayer reads all rows of the streams")
        n = self.norm
        y = torch.empty(x.shape[0], n.size, dtype=out_dtype, device=x.device)
        kernels.hc_read(y, x, self.in_w, n.w, n.eps, n.offset, self.block.streams)
        return y


@register_part("block", "hyper")
class HyperBlock(Block):
    """Parameters: ``streams``, ``hidden_size``; optional ``connections``: for the mixer and for the feed-forward a
    dictionary {``in`` ([streams]), ``mix`` ([streams, streams], indexed [from, to]), ``out`` ([streams])} of tensor
    names (absent: in = out = 1 and mix the identity, which wants one stream); optional ``scales``: the tensor names
    of the two per-channel layer scales (either may be None).  Norm roles ``pre_mixer`` and ``pre_feed_forward``
    (``rms_norm``)."""
    roles = ("pre_mixer", "pre_feed_forward")

    def __init__(self, params, ctx, mixer, feed_forward, norms):
        if not feed_forward.present:
            self.roles = ("pre_mixer",)
        super().__init__(params, ctx, mixer, feed_forward, norms)
        self.streams = int(self.param("streams"))
        self.hidden = int(self.param("hidden_size"))
        if not 1 <= self.streams <= kernels.HC_MAX_STREAMS:
            raise ConfigError(f"hyper: 1 to {kernels.HC_MAX_STREAMS} streams, got {self.streams}")
        self.names = self.params.get("connections")
        if self.names is None and self.streams != 1:
            raise ConfigError("hyper: several streams need their connection weights")
        self.scale_names = tuple(self.params.get("scales") or (None, None))
        for n in norms.values():
            if not isinstance(n, RmsNorm):
                raise ConfigError("hyper: the norms in front of the sublayers are of the kind rms_norm")
        self.halves = 2 if feed_forward.present else 1
        self.conn = [None, None]
        self.scale = [None, None]
        self.readers = [StreamReader(self, 0), StreamReader(self, 1)]

    def weight_decls(self):
        S, decls = self.streams, super().weight_decls()
        for q in range(self.halves):
            if self.names is not None:
                nm = self.names[q]
                decls += [WeightDecl(nm["in"], (S,), "share"), WeightDecl(nm["mix"], (S, S), "mixing"),
                          WeightDecl(nm["out"], (S,), "gain")]
            if self.scale_names[q]:
                decls.append(WeightDecl(self.scale_names[q], (self.hidden,), "gain"))
        return decls

    def load(self, weights):
        super().load(weights)
        f32, S, dev = torch.float32, self.streams, self.ctx.device
        for q in range(self.halves):
            if self.names is not None:
                nm = self.names[q]
                self.conn[q] = tuple(weights[nm[k]].to(f32).contiguous() for k in ("in", "mix", "out"))
            else:
                self.conn[q] = (torch.ones(S, dtype=f32, device=dev), torch.eye(S, dtype=f32, device=dev),
                                torch.ones(S, dtype=f32, device=dev))
            if self.scale_names[q]:
                self.scale[q] = weights[self.scale_names[q]].to(f32).contiguous()

    def decode_bytes(self, lens) -> int:
        # the streams are read and written once a sublayer
        return super().decode_bytes(lens) + self.halves * len(lens) * 2 * 4 * self.streams * self.hidden

    def first_norm(self):
        return self.readers[0]

    def _write(self, q: int, x, result, then, dt):
        """Rewrite the streams from sublayer q's result; returns what ``then`` reads of the new streams."""
        terms = as_terms(result)
        if len(terms) > 2:
            total = torch.zeros(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
            kernels.add_scaled_rmsnorm(total, terms)
            terms = [(total, 1.0)]
        _, mix, out_w = self.conn[q]
        fused = isinstance(then, StreamReader)
        y = torch.empty(x.shape[0], self.hidden, dtype=dt, device=x.device) if fused else None
        n = then.norm if fused else None
        kernels.hc_write(x, terms, mix, out_w, self.streams, scale=self.scale[q], y=y,
                         in_next=then.in_w if fused else None, w_next=n.w if fused else None,
                         eps=n.eps if fused else 0.0, offset=n.offset if fused else 0.0)
        if fused or then is None:
            return y
        return then.forward(x, dt)

    def forward(self, x, batch, view, normed=None, next_pre=None):
        dt = self.ctx.compute_dtype
        if x.shape[1] != self.streams * self.hidden:
            raise ConfigError(f"hyper: the stream holds {x.shape[1]} values a token, not {self.streams} x {self.hidden}")
        h = normed if normed is not None else self.readers[0].forward(x, dt)
        a = self.mixer.forward(h, batch, view)
        if not self.feed_forward.present:
            return self._write(0, x, a, next_pre, dt)
        h = self._write(0, x, a, self.readers[1], dt)
        return self._write(1, x, self.feed_forward.forward(h, batch), next_pre, dt)
