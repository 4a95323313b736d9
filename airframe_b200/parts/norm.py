"""Norms of the residual stream.

``rms_norm``: y = x * rsqrt(mean(x^2) + eps) * (offset + w).
``tanh_norm``: y = tanh(alpha x) w + b with a scalar alpha: no mean and no
variance, so it is elementwise and a row needs no reduction.
``as_is``: y = x in the compute dtype: what a sublayer is given that reads the
stream itself (a norm only behind it); a residual kernel writes it beside the sum.

Reference: ``src/backend/bindless/sh_layer_v1.wgsl:426-451``,
``src/backend/bindless/sh_rmsnorm.wgsl:69-93``; post norms fused with the
residual sum as x + norm(a) instead of the reference's add-then-correct
(``sh_layer_v1.wgsl:811-813,834-849``).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import Norm, register_part
from .linear import PartialSums, as_terms


@register_part("norm", "rms_norm")
class RmsNorm(Norm):
    """Parameters: ``weight`` (tensor name), ``size``, ``eps``, ``weight_offset``."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.name = self.param("weight")
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))
        self.offset = float(self.param("weight_offset"))
        self.w = None

    def weight_decls(self):
        return [WeightDecl(self.name, (self.size,), "norm")]

    def load(self, weights):
        # statistics and the (offset + w) factor are 32-bit in both precisions
        self.w = weights[self.name].to(torch.float32).contiguous()

    def decode_bytes(self, lens) -> int:
        return 4 * self.size

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty(n, self.size, dtype=out_dtype, device=x.device)
        kernels.rmsnorm(y, x, self.w, self.eps, self.offset, rows)
        return y

    def add_normed(self, x, a, then=None, out_dtype=None):
        """x += this norm of ``a`` (a tensor, partial sums, or a weighted sum of those, which is taken in 32
        bits under the norm); with ``then`` its output for the new x, out of the same kernel where that
        kernel exists (another ``rms_norm``, or ``as_is``)."""
        terms = as_terms(a)
        plain = len(terms) == 1 and terms[0][1] == 1.0
        same = isinstance(then, RmsNorm) and then.offset == self.offset
        if not plain or isinstance(then, AsIs) or (isinstance(then, RmsNorm) and not same):
            fused = then is None or isinstance(then, (RmsNorm, AsIs))
            y = None
            alias = isinstance(then, AsIs) and out_dtype == torch.float32      # (the 32-bit stream is its own copy)
            if then is not None and fused and not alias:
                y = torch.empty(x.shape[0], self.size, dtype=out_dtype, device=x.device)
            nxt = then if isinstance(then, RmsNorm) else None
            kernels.add_normed_terms(x, terms, self.w, self.eps, self.offset, y=y,
                                     w_next=nxt.w if nxt is not None else None,
                                     eps_next=nxt.eps if nxt is not None else 0.0,
                                     offset_next=nxt.offset if nxt is not None else 0.0)
            if alias:
                return x
            return y if fused else then.forward(x, out_dtype)
        a = terms[0][0]                 # (one term with a scale of 1, whatever form it came in)
        n_parts = a.shape[0] if a.dim() == 3 else 1
        if then is not None and not (isinstance(then, RmsNorm) and then.offset == self.offset):
            kernels.add_rmsnorm(x, a, self.w, self.eps, self.offset, n_parts=n_parts)
            return then.forward(x, out_dtype)
        y = None
        if then is not None:
            y = torch.empty(x.shape[0], self.size, dtype=out_dtype, device=x.device)
        kernels.add_rmsnorm(x, a, self.w, self.eps, self.offset, y=y,
                            w_next=then.w if then is not None else None,
                            eps_next=then.eps if then is not None else 0.0, n_parts=n_parts)
        return y

    def after_add(self, x, a, out_dtype):
        """x += a (a tensor, partial sums or a weighted sum of them) and this norm
        of the new x, in one kernel."""
        y = torch.empty(x.shape[0], self.size, dtype=out_dtype, device=x.device)
        kernels.add_scaled_rmsnorm(x, as_terms(a), y=y, w_next=self.w, eps=self.eps, offset=self.offset)
        return y


@register_part("norm", "tanh_norm")
class TanhNorm(Norm):
    """y = tanh(alpha x) w + b.  Parameters: ``weight``, ``bias``, ``alpha`` (tensor names; alpha a scalar), ``size``."""
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.names = (self.param("weight"), self.param("bias"), self.param("alpha"))
        self.size = int(self.param("size"))
        self.w = self.b = None
        self.alpha = 0.0

    def weight_decls(self):
        w, b, a = self.names
        return [WeightDecl(w, (self.size,), "gain"), WeightDecl(b, (self.size,), "norm"), WeightDecl(a, (), "gain")]

    def load(self, weights):
        w, b, a = self.names
        self.w = weights[w].to(torch.float32).contiguous()
        self.b = weights[b].to(torch.float32).contiguous()
        self.alpha = float(weights[a].to(torch.float32).item())      # (read once, when the model loads)

    def decode_bytes(self, lens) -> int:
        return 8 * self.size

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty(n, self.size, dtype=out_dtype, device=x.device)
        kernels.tanh_norm(y, x, self.w, self.b, self.alpha, rows)
        return y

    def add_normed(self, x, a, then=None, out_dtype=None):
        """x += this norm of ``a``; with ``then`` (a norm of this kind) its output for the new x comes out of the
        same kernel."""
        if isinstance(a, PartialSums):
            a = a.parts
        if then is not None and not isinstance(then, TanhNorm):
            kernels.add_tanh_norm(x, a, self.w, self.b, self.alpha)
            return then.forward(x, out_dtype)
        y = None
        if then is not None:
            y = torch.empty(x.shape[0], self.size, dtype=out_dtype, device=x.device)
        kernels.add_tanh_norm(x, a, self.w, self.b, self.alpha, y=y, w_next=then.w if then is not None else None,
                              b_next=then.b if then is not None else None,
                              alpha_next=then.alpha if then is not None else 0.0)
        return y


@register_part("norm", "as_is")
class AsIs(Norm):
    """No norm at all: the residual stream as it stands, in the dtype asked for.  Parameters: ``size``.  It
    stands where a block wants "the norm in front of a sublayer" and the design has none there; the residual
    kernels of the other norms write its output beside their sum (``add_normed(..., then=)``)."""
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size = int(self.param("size"))

    def forward(self, x, out_dtype, rows=None):
        if rows is None and out_dtype == torch.float32:
            return x                    # (the sublayer reads the stream itself; it is rewritten only once the sublayer is done)
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty(n, self.size, dtype=out_dtype, device=x.device)
        kernels.cast_rows(y, x, rows)
        return y

    def add_normed(self, x, a, then=None, out_dtype=None):
        if then is not None:
            return then.after_add(x, a, out_dtype)
        kernels.add_scaled_rmsnorm(x, as_terms(a))
        return None

    def after_add(self, x, a, out_dtype):
        kernels.add_scaled_rmsnorm(x, as_terms(a))
        return self.forward(x, out_dtype)
