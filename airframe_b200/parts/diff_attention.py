"""Differential attention: every head attends twice over the same values, with
two sets of queries and keys ("maps"), and the second result is subtracted from
the first:

    a_m = softmax(cap(scale q_m k_m^T)) v   (m = 1, 2; causal, cap(s) = softcap tanh(s / softcap))
    o   = a_1 - lambda a_2,  o <- o / sqrt(mean(o^2) + eps) * (1 - diff)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff      (one number for the layer)

Query head h reads key/value head h // (heads / kv_heads); a q row holds its head's
[map 1 | map 2], a k row likewise.  Options, each a parameter: biases of the q, k, v
and output projections; a short causal convolution over time on every channel of q,
k and v (directly behind the projection; its last taps - 1 inputs are the sequence's
state); a query temperature 1 + coef ln(floor((p + 1) / every) + 1) at position p;
the softcap; an output gate sigmoid(W_g h) per element of the concatenated heads.

The two maps run through the library's grouped attention kernels as heads of their
own (see ``kernels.conv_pack`` for the order), so prompts run on the tensor-core
kernels and decode steps on the split kernel over the paged cache wherever the head
size allows; the cache then holds a group's values once per map.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import WeightDecl
from .base import KVNeed, Mixer, StateNeed, register_part
from .linear import linear, linear_split


@register_part("mixer", "diff_attention")
class DiffAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim`` (of one map's queries and keys),
    ``value_dim``, ``scale``, ``diff``, ``eps``, ``softcap`` (0 or None = off), ``window`` (None = all keys),
    ``weights``: tensor names for ``q, k, v, o, lq1, lk1, lq2, lk2`` and optionally ``q_bias, k_bias, v_bias`` (all or
    none), ``o_bias``, ``g`` (the output gate), ``q_conv, k_conv, v_conv`` ([channels, taps], all or none);
    optional ``taps`` (with the convolutions), ``q_temp``: {``coef``, ``every``}; optional ``wide_output``
    (default true)."""
    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.H = int(self.param("num_heads"))
        self.G = int(self.param("num_kv_heads"))
        self.d = int(self.param("head_dim"))
        self.dv = int(self.param("value_dim"))
        self.scale = float(self.param("scale"))
        self.diff = float(self.param("diff"))
        self.eps = float(self.param("eps"))
        self.softcap = float(self.params.get("softcap") or 0.0)
        w = self.params.get("window")
        self.window = int(w) if w else None
        if self.H % self.G:
            raise ConfigError(f"diff_attention: {self.H} heads are not a multiple of {self.G} kv heads")
        self.names = dict(self.param("weights"))
        missing = [r for r in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2") if not self.names.get(r)]
        if missing:
            raise ConfigError(f"diff_attention: parameter 'weights' names no tensor for {missing}")
        bias = [bool(self.names.get(r)) for r in ("q_bias", "k_bias", "v_bias")]
        conv = [bool(self.names.get(r)) for r in ("q_conv", "k_conv", "v_conv")]
        if any(bias) != all(bias) or any(conv) != all(conv):
            raise ConfigError("diff_attention: biases (and convolutions) for all of q, k and v, or for none")
        self.has_bias, self.has_conv = all(bias), all(conv)
        self.taps = int(self.params.get("taps") or 1) if self.has_conv else 1
        if self.has_conv and self.taps < 1:
            raise ConfigError("diff_attention: a convolution has at least the token's own tap")
        qt = self.params.get("q_temp")
        self.temp_coef, self.temp_every = (float(qt["coef"]), int(qt["every"])) if qt else (0.0, 0)
        if qt and self.temp_every < 1:
            raise ConfigError("diff_attention: q_temp.every must be >= 1")
        self.cq, self.ck, self.cv = self.H * 2 * self.d, self.G * 2 * self.d, self.G * self.dv
        self.channels = self.cq + self.ck + self.cv
        # bfloat16 heads go to the tensor-core attention kernels where padding them with zeros up to a size those
        # take costs at most twice the larger of the two head sizes; else the plain kernels take them as they are
        self.pk, self.pv = self.d, self.dv
        big = max(self.d, self.dv)
        if ctx.compute_dtype == torch.bfloat16:
            fit = next((p for p in kernels.FAST_HEAD_SIZES if p >= big), 0)
            if fit and fit <= 2 * big:
                self.pk = self.pv = fit
        # the output projection takes one more input column that is always 1: its weight there is the bias
        # (columns up to a multiple of eight, so that the tensor-core product takes the rows)
        self.o_in = self.H * self.dv
        if self.names.get("o_bias"):
            self.o_in = -(-(self.H * self.dv + 1) // 8) * 8
        self.lam = 0.0

    def kv_need(self):
        return KVNeed(2 * self.G, self.pk, self.window, None if self.pv == self.pk else self.pv)

    def state_need(self):
        return StateNeed((self.taps - 1, self.channels), "float32") if self.taps > 1 else None

    def weight_decls(self):
        nm, h = self.names, self.hidden
        decls = [WeightDecl(nm["q"], (self.cq, h)), WeightDecl(nm["k"], (self.ck, h)), WeightDecl(nm["v"], (self.cv, h)),
                 WeightDecl(nm["o"], (h, self.H * self.dv)),
                 *(WeightDecl(nm[r], (self.d,), "norm") for r in ("lq1", "lk1", "lq2", "lk2"))]
        if self.has_bias:
            decls += [WeightDecl(nm["q_bias"], (self.cq,), "norm"), WeightDecl(nm["k_bias"], (self.ck,), "norm"),
                      WeightDecl(nm["v_bias"], (self.cv,), "norm")]
        if self.has_conv:
            decls += [WeightDecl(nm["q_conv"], (self.cq, self.taps), "gain"), WeightDecl(nm["k_conv"], (self.ck, self.taps), "gain"),
                      WeightDecl(nm["v_conv"], (self.cv, self.taps), "gain")]
        if nm.get("o_bias"):
            decls.append(WeightDecl(nm["o_bias"], (h,), "norm"))
        if nm.get("g"):
            decls.append(WeightDecl(nm["g"], (self.H * self.dv, h)))
        return decls

    def load(self, weights):
        nm, dt, f32 = self.names, self.ctx.compute_dtype, torch.float32
        mats = [weights[nm["q"]], weights[nm["k"]], weights[nm["v"]]]
        if nm.get("g"):
            mats.append(weights[nm["g"]])           # the gate's logits ride behind [q | k | v] in the same product
        pad = (-sum(m.shape[0] for m in mats)) % 4
        if pad:
            mats.append(torch.zeros(pad, self.hidden, dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).to(dt).contiguous()
        self.bias = (torch.cat([weights[nm[r]].to(f32).reshape(-1) for r in ("q_bias", "k_bias", "v_bias")]).contiguous()
                     if self.has_bias else None)
        self.taps_w = None
        if self.has_conv:
            self.taps_w = torch.cat([weights[nm[r]].to(f32) for r in ("q_conv", "k_conv", "v_conv")], dim=0).t().contiguous()
        w_o = weights[nm["o"]].to(dt)
        if self.o_in != self.H * self.dv:
            wide = torch.zeros(self.hidden, self.o_in, dtype=dt, device=w_o.device)
            wide[:, : self.H * self.dv] = w_o
            wide[:, self.H * self.dv] = weights[nm["o_bias"]].to(dt)
            w_o = wide
        self.w_o = w_o.contiguous()
        f64 = torch.float64
        dots = [float((weights[nm[a]].to(f64) * weights[nm[b]].to(f64)).sum()) for a, b in (("lq1", "lk1"), ("lq2", "lk2"))]
        self.lam = math.exp(dots[0]) - math.exp(dots[1]) + self.diff

    def _el(self) -> int:
        return 4 if self.ctx.compute_dtype == torch.float32 else 2

    def _visible(self, pos: int) -> int:
        return min(pos + 1, self.window) if self.window else pos + 1

    def decode_bytes(self, lens) -> int:
        weights = (self.w_in.numel() + self.w_o.numel()) * self._el()
        kv_row = 2 * self.G * (self.pk + self.pv) * self._el()
        state = 2 * 4 * (self.taps - 1) * self.channels
        return weights + sum(kv_row * self._visible(n - 1) + state for n in lens)

    def score_flops(self, lens) -> int:
        pairs = 0
        for n in lens:
            w = self.window
            pairs += n * (n + 1) // 2 if not w or n <= w else w * (w + 1) // 2 + (n - w) * w
        return 2 * pairs * 2 * self.H * (self.d + self.dv)

    def prefill_flops(self, lens) -> int:
        return 2 * sum(lens) * (self.w_in.numel() + self.w_o.numel()) + self.score_flops(lens)

    def forward(self, x, batch, view):
        T, H, G, pk, pv = x.shape[0], self.H, self.G, self.pk, self.pv
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        qkv = torch.empty(T, (2 * H + 2 * G) * pk + 2 * G * pv, dtype=x.dtype, device=x.device)
        kernels.conv_pack(qkv, proj, batch, H, G, self.d, self.dv, pk, pv, bias=self.bias, taps_w=self.taps_w,
                          history=view.state, temp_coef=self.temp_coef, temp_every=self.temp_every,
                          kv=view.kv if view.writes else None)
        nq, nkv = 2 * H, 2 * G
        q = qkv[:, : nq * pk]
        k = qkv[:, nq * pk: (nq + nkv) * pk]
        v = qkv[:, (nq + nkv) * pk:]
        ctx = torch.empty(T, nq * pv, dtype=x.dtype, device=x.device)
        window = self.window or 0
        if batch.is_prefill:
            if not view.writes:
                k, v = batch.step_kv[view.cache_id]
            elif view.keep_step_kv:
                batch.step_kv[view.cache_id] = (k.clone(), v.clone())
            kernels.attn_prefill(ctx, q, k, v, batch, nq, nkv, pk, self.scale, self.softcap, window, dv=pv)
        else:
            kernels.attn_decode(ctx, q, view.kv, batch, nq, nkv, pk, self.scale, self.softcap, window, dv=pv)
        y = torch.empty(T, self.o_in, dtype=x.dtype, device=x.device)
        gate = proj[:, self.channels: self.channels + H * self.dv] if self.names.get("g") else None
        kernels.diff_join(y, ctx, gate, H, G, self.dv, pv, self.lam, self.eps, 1.0 - self.diff,
                          ones=1 if self.o_in != H * self.dv else 0)
        return linear_split(y, self.w_o, wide=bool(self.params.get("wide_output", True)))
