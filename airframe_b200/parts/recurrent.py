"""Mixers that keep a state of fixed size per sequence instead of keys and
values.  The state lives in the cache's per-sequence state (32-bit floats, zero
when a sequence starts) and is carried from step to step; a prompt in one step
and the same tokens one by one run the same recurrence token after token.

``general_delta``: the generalized delta rule.  Per head, with r, k, v of the
token, a decay w per key channel, a removal rate a per key channel and the unit
key u = k / sqrt(|k|^2 + key_eps):

    S <- diag(w) S - (a * u)(u^T S) + k v^T        o = S^T r

(the decay and the removal act on the state before the token).  w = exp(-decay_scale * sigmoid(W2 tanh(W1 h) + w0)),
a = sigmoid(Wa h + ba).  Each head's o is divided by its root mean square, times a
weight vector (no offset), times sigmoid(Wg h), then the output projection.

``lightning_attention``: linear attention with a fixed decay per head:
q, k, v = silu of their projections, S <- decay_h S + k v^T, o = S^T q; the heads
together are RMS-normed with a weight vector (no offset), times sigmoid(Wg h), then projected.

``mingru``: a gated recurrence over a vector: z = sigmoid(Wz h + bz),
c = Wx h + bx, candidate = c + 1/2 where c >= 0 and sigmoid(c) below,
S <- (1 - z) S + z * candidate, output Wo (S * silu(Wg h)).

``rglru``: a real-gated linear recurrence behind a short causal convolution (the
recurrent block of Griffin): y = gelu_tanh(Wy h + by), u = conv(Wx h + bx) per
channel; with the channels in ``blocks`` equal parts and block-diagonal gate
matrices, r = sigmoid(Wa u + ba), i = sigmoid(Wi u + bi), a = exp(-decay_rate r
softplus(lam)), S <- a S + sqrt(1 - a^2) i u, output Wo (S * y).  The state of a
sequence is S and the convolution's last taps - 1 inputs.

Every projection of a mixer is one product into 32-bit rows; what enters a
recurrence (decays, gates, unit keys) is worked out in 32 bits from them.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import WeightDecl
from .base import Mixer, StateNeed, register_part
from .linear import linear, linear_split


def _el(ctx) -> int:
    return 4 if ctx.compute_dtype == torch.float32 else 2


class _StateMixer(Mixer):
    """What the three have in common: named tensors, one packed projection, and an
    output projection whose result goes to the residual sum in 32 bits (optional
    parameter ``wide_output``, default true)."""
    graph_safe = True

    @property
    def wide(self) -> bool:
        return bool(self.params.get("wide_output", True))

    def _names(self, roles):
        names = self.param("weights")
        missing = [r for r in roles if r not in names]
        if missing:
            raise ConfigError(f"{self.kind}: parameter 'weights' names no tensor for {missing}")
        return {r: names[r] for r in roles}

    def _pack(self, weights, roles):
        """The rows of the named matrices one under the other (each section padded to a multiple
        of four rows so that sections of 32-bit output rows start on 16 bytes) and where each starts."""
        dt = self.ctx.compute_dtype
        mats, offsets, at = [], {}, 0
        for r in roles:
            w = weights[self.names[r]].to(dt)
            offsets[r] = at
            pad = (-w.shape[0]) % 4
            if pad:
                w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=dt, device=w.device)])
            mats.append(w)
            at += w.shape[0]
        return torch.cat(mats, dim=0).contiguous(), offsets


@register_part("mixer", "general_delta")
class GeneralDelta(_StateMixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (keys and values),
    ``eps`` (of the output norm), ``weights``: tensor names for ``r, k, v, g, a, a_bias,
    w1, w2, w0, norm, o``; optional ``decay_rank`` (rows of w1; read from the tensor when
    absent), ``decay_scale`` (default exp(-1/2)), ``key_eps`` (default 1e-6)."""
    ROLES = ("r", "k", "v", "g", "a", "a_bias", "w1", "w2", "w0", "norm", "o")

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.hd = int(self.param("head_dim"))
        self.eps = float(self.param("eps"))
        rank = self.params.get("decay_rank")
        self.rank = int(rank) if rank is not None else None
        self.decay_scale = float(self.params.get("decay_scale", math.exp(-0.5)))
        self.key_eps = float(self.params.get("key_eps", 1e-6))
        self.names = self._names(self.ROLES)
        self.n = self.heads * self.hd

    def state_need(self):
        return StateNeed((self.heads, self.hd, self.hd), "float32")      # [head][value column][key channel]

    def weight_decls(self):
        n, h, nm = self.n, self.hidden, self.names
        return [*(WeightDecl(nm[r], (n, h)) for r in ("r", "k", "v", "g", "a")),
                WeightDecl(nm["a_bias"], (n,), "norm"), WeightDecl(nm["w1"], (self.rank, h)),
                WeightDecl(nm["w2"], (n, self.rank)), WeightDecl(nm["w0"], (n,), "norm"),
                WeightDecl(nm["norm"], (n,), "norm"), WeightDecl(nm["o"], (h, n))]

    def load(self, weights):
        nm = self.names
        self.rank = weights[nm["w1"]].shape[0]
        if weights[nm["w2"]].shape[1] != self.rank:
            raise ConfigError(f"general_delta: {nm['w1']} has {self.rank} rows, {nm['w2']} has "
                              f"{weights[nm['w2']].shape[1]} columns")
        self.w_in, self.off = self._pack(weights, ("r", "k", "v", "g", "a", "w1"))
        f32 = torch.float32
        self.a_bias = weights[nm["a_bias"]].to(f32).contiguous()
        self.w0 = weights[nm["w0"]].to(f32).contiguous()
        self.w2t = weights[nm["w2"]].to(f32).t().contiguous()      # [rank, heads * dim]: channels side by side
        self.norm_w = weights[nm["norm"]].to(f32).contiguous()
        self.w_o = weights[nm["o"]].to(self.ctx.compute_dtype).contiguous()

    def decode_bytes(self, lens) -> int:
        weights = (self.w_in.numel() + self.w_o.numel()) * _el(self.ctx) + 4 * self.w2t.numel()
        return weights + len(lens) * 2 * 4 * self.heads * self.hd * self.hd      # the state, read and written

    def prefill_flops(self, lens) -> int:
        T = sum(lens)
        return 2 * T * (self.w_in.numel() + self.w_o.numel()) + T * self.heads * 7 * self.hd * self.hd

    def forward(self, x, batch, view):
        T, n, off = x.shape[0], self.n, self.off
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        pre = torch.empty(T, 3, n, dtype=torch.float32, device=x.device)
        kernels.delta_prep(pre, proj, off["k"], off["a"], off["w1"], self.a_bias, self.w0, self.w2t, self.heads,
                           self.hd, self.decay_scale, self.key_eps)
        o = torch.empty(T, n, dtype=torch.float32, device=x.device)
        kernels.state_scan("delta", o, proj[:, off["r"]: off["r"] + n], proj[:, off["k"]: off["k"] + n],
                           proj[:, off["v"]: off["v"] + n], view.state, batch, self.heads, self.hd, self.hd,
                           w=pre[:, 0], u=pre[:, 1], au=pre[:, 2])
        y = torch.empty(T, n, dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(y, o, self.norm_w, proj[:, off["g"]: off["g"] + n], self.hd, self.eps)
        return linear_split(y, self.w_o, wide=self.wide)


@register_part("mixer", "lightning_attention")
class LightningAttention(_StateMixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (queries and keys),
    ``value_dim``, ``decay`` (one factor per head), ``eps`` (of the output norm),
    ``weights``: tensor names for ``q, k, v, g, norm, o``."""
    ROLES = ("q", "k", "v", "g", "norm", "o")

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.dk = int(self.param("head_dim"))
        self.dv = int(self.param("value_dim"))
        self.eps = float(self.param("eps"))
        decay = self.param("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != self.heads:
            raise ConfigError(f"lightning_attention: 'decay' must list one factor for each of the {self.heads} heads")
        self.decay_host = torch.tensor([float(d) for d in decay], dtype=torch.float64).to(torch.float32)
        self.names = self._names(self.ROLES)

    def state_need(self):
        return StateNeed((self.heads, self.dv, self.dk), "float32")

    def weight_decls(self):
        nk, nv, h, nm = self.heads * self.dk, self.heads * self.dv, self.hidden, self.names
        return [WeightDecl(nm["q"], (nk, h)), WeightDecl(nm["k"], (nk, h)), WeightDecl(nm["v"], (nv, h)),
                WeightDecl(nm["g"], (nv, h)), WeightDecl(nm["norm"], (nv,), "norm"), WeightDecl(nm["o"], (h, nv))]

    def load(self, weights):
        nm = self.names
        self.w_in, self.off = self._pack(weights, ("q", "k", "v", "g"))
        self.norm_w = weights[nm["norm"]].to(torch.float32).contiguous()
        self.w_o = weights[nm["o"]].to(self.ctx.compute_dtype).contiguous()
        self.decay = self.decay_host.to(self.ctx.device)

    def decode_bytes(self, lens) -> int:
        return ((self.w_in.numel() + self.w_o.numel()) * _el(self.ctx)
                + len(lens) * 2 * 4 * self.heads * self.dk * self.dv)

    def prefill_flops(self, lens) -> int:
        T = sum(lens)
        return 2 * T * (self.w_in.numel() + self.w_o.numel()) + T * self.heads * 4 * self.dk * self.dv

    def forward(self, x, batch, view):
        T, off = x.shape[0], self.off
        nk, nv = self.heads * self.dk, self.heads * self.dv
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        o = torch.empty(T, nv, dtype=torch.float32, device=x.device)
        kernels.state_scan("decay", o, proj[:, off["q"]: off["q"] + nk], proj[:, off["k"]: off["k"] + nk],
                           proj[:, off["v"]: off["v"] + nv], view.state, batch, self.heads, self.dk, self.dv,
                           decay=self.decay, silu=True)
        y = torch.empty(T, nv, dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(y, o, self.norm_w, proj[:, off["g"]: off["g"] + nv], nv, self.eps)
        return linear_split(y, self.w_o, wide=self.wide)


@register_part("mixer", "mingru")
class MinGru(_StateMixer):
    """Parameters: ``hidden_size``, ``width`` (of the state), ``weights``: tensor
    names for ``z, z_bias, x, x_bias, g, o``."""
    ROLES = ("z", "z_bias", "x", "x_bias", "g", "o")

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.width = int(self.param("width"))
        self.names = self._names(self.ROLES)

    def state_need(self):
        return StateNeed((self.width,), "float32")

    def weight_decls(self):
        w, h, nm = self.width, self.hidden, self.names
        return [WeightDecl(nm["z"], (w, h)), WeightDecl(nm["z_bias"], (w,), "norm"), WeightDecl(nm["x"], (w, h)),
                WeightDecl(nm["x_bias"], (w,), "norm"), WeightDecl(nm["g"], (w, h)), WeightDecl(nm["o"], (h, w))]

    def load(self, weights):
        nm = self.names
        self.w_in, self.off = self._pack(weights, ("z", "x", "g"))
        self.z_bias = weights[nm["z_bias"]].to(torch.float32).contiguous()
        self.x_bias = weights[nm["x_bias"]].to(torch.float32).contiguous()
        self.w_o = weights[nm["o"]].to(self.ctx.compute_dtype).contiguous()

    def decode_bytes(self, lens) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * _el(self.ctx) + len(lens) * 2 * 4 * self.width

    def prefill_flops(self, lens) -> int:
        return 2 * sum(lens) * (self.w_in.numel() + self.w_o.numel())

    def forward(self, x, batch, view):
        off = self.off
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        y = torch.empty(x.shape[0], self.width, dtype=x.dtype, device=x.device)
        kernels.gated_scan(y, proj, off["z"], off["x"], off["g"], self.z_bias, self.x_bias, view.state, batch)
        return linear_split(y, self.w_o, wide=self.wide)


@register_part("mixer", "rglru")
class RgLru(_StateMixer):
    """Parameters: ``hidden_size``, ``width`` (of the state), ``blocks`` (of the gates' block-diagonal
    matrices), ``taps`` (of the convolution), ``weights``: tensor names for ``y, y_bias, x, x_bias, conv
    ([width, taps], the last column on the current token), conv_bias, a ([blocks, width / blocks, width /
    blocks], [out, in]), a_bias ([blocks, width / blocks]), i, i_bias, lam, o``; optional ``decay_rate``
    (default 8)."""
    ROLES = ("y", "y_bias", "x", "x_bias", "conv", "conv_bias", "a", "a_bias", "i", "i_bias", "lam", "o")

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.width = int(self.param("width"))
        self.blocks = int(self.param("blocks"))
        self.taps = int(self.param("taps"))
        self.decay_rate = float(self.params.get("decay_rate", 8.0))
        if self.blocks < 1 or self.width % self.blocks:
            raise ConfigError(f"rglru: {self.width} channels do not come in {self.blocks} equal blocks")
        if self.taps < 1:
            raise ConfigError("rglru: the convolution has at least the current token's tap")
        self.names = self._names(self.ROLES)

    def state_need(self):
        return StateNeed((self.taps, self.width), "float32")      # row 0: S; then the convolution's last inputs

    def weight_decls(self):
        w, h, b, nm = self.width, self.hidden, self.blocks, self.names
        bw = w // b
        return [WeightDecl(nm["y"], (w, h)), WeightDecl(nm["y_bias"], (w,), "norm"),
                WeightDecl(nm["x"], (w, h)), WeightDecl(nm["x_bias"], (w,), "norm"),
                WeightDecl(nm["conv"], (w, self.taps), "gain"), WeightDecl(nm["conv_bias"], (w,), "norm"),
                WeightDecl(nm["a"], (b, bw, bw)), WeightDecl(nm["a_bias"], (b, bw), "norm"),
                WeightDecl(nm["i"], (b, bw, bw)), WeightDecl(nm["i_bias"], (b, bw), "norm"),
                WeightDecl(nm["lam"], (w,), "gain"), WeightDecl(nm["o"], (h, w))]

    def load(self, weights):
        nm, f32, dt = self.names, torch.float32, self.ctx.compute_dtype
        self.w_in, self.off = self._pack(weights, ("y", "x"))
        self.y_bias = weights[nm["y_bias"]].to(f32).contiguous()
        self.x_bias = weights[nm["x_bias"]].to(f32).contiguous()
        self.conv_w = weights[nm["conv"]].to(f32).t().contiguous()       # [taps, width]: a warp reads a tap of 32 channels in one line
        self.conv_b = weights[nm["conv_bias"]].to(f32).contiguous()
        self.w_a = weights[nm["a"]].to(dt).contiguous()
        self.w_i = weights[nm["i"]].to(dt).contiguous()
        self.a_bias = weights[nm["a_bias"]].to(f32).reshape(-1).contiguous()
        self.i_bias = weights[nm["i_bias"]].to(f32).reshape(-1).contiguous()
        # decay_rate * softplus(lam), once, from the stored values (worked out in 64 bits, kept in 32)
        self.rate = (self.decay_rate * torch.nn.functional.softplus(weights[nm["lam"]].to(torch.float64))).to(f32).contiguous()
        self.w_o = weights[nm["o"]].to(dt).contiguous()

    def decode_bytes(self, lens) -> int:
        weights = (self.w_in.numel() + self.w_o.numel() + self.w_a.numel() + self.w_i.numel()) * _el(self.ctx)
        return weights + len(lens) * 2 * 4 * self.taps * self.width

    def prefill_flops(self, lens) -> int:
        return 2 * sum(lens) * (self.w_in.numel() + self.w_o.numel() + self.w_a.numel() + self.w_i.numel())

    def forward(self, x, batch, view):
        T, w, off, f32 = x.shape[0], self.width, self.off, torch.float32
        proj = linear(x, self.w_in, out_dtype=f32)
        u = torch.empty(T, w, dtype=f32, device=x.device)
        # many rows in bfloat16: the gates' block-diagonal products on the tensor cores, from u rounded as
        # every product's input is; few rows (a decode step) or 32-bit: on the CUDA cores from u itself
        fast = T >= kernels.GATE_TC_ROWS and kernels.gate_rows_tc_supported(u, self.w_a)
        u16 = torch.empty(T, w, dtype=torch.bfloat16, device=x.device) if fast else None
        kernels.conv_rows(u, proj, off["x"], self.x_bias, self.conv_w, self.conv_b, view.state, batch, u16=u16)
        decay = torch.empty(T, w, dtype=f32, device=x.device)
        inp = torch.empty(T, w, dtype=f32, device=x.device)
        if fast:
            kernels.gate_rows_tc(decay, inp, u, u16, self.w_a, self.w_i, self.a_bias, self.i_bias, self.rate)
        else:
            kernels.gate_rows(decay, inp, u, self.w_a, self.w_i, self.a_bias, self.i_bias, self.rate)
        y = torch.empty(T, w, dtype=x.dtype, device=x.device)
        kernels.decay_scan(y, decay, inp, proj, off["y"], off["x"], self.y_bias, self.x_bias, view.state, batch)
        return linear_split(y, self.w_o, wide=self.wide)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(_StateMixer):
    """Linear attention whose state decays by a factor per key channel and token:

        q = query_scale W_q h, k = W_k h, v = W_v h, alpha = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau)
        S <- diag(alpha) S + k v^T (per head, from zero), o = S^T q

    each head's o is divided by its root mean square (``eps`` inside the root), times a weight of ``value_dim``
    values that the heads share, times silu(W_g h), then the output projection.

    Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (queries and keys), ``value_dim``, ``tau``, ``eps``,
    ``weights``: tensor names for ``q, k, v, g, a1, a2, a2_bias, norm, o``; optional ``query_scale`` (default
    head_dim^-1/2), ``decay_rank`` (rows of a1; read from the tensor when absent), ``gate`` ("silu", the default, or
    "sigmoid"), ``chunked_scan`` (default true: a step of few long prompts scans chunks of them side by side)."""
    ROLES = ("q", "k", "v", "g", "a1", "a2", "a2_bias", "norm", "o")

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.dk = int(self.param("head_dim"))
        self.dv = int(self.param("value_dim"))
        self.tau = float(self.param("tau"))
        self.eps = float(self.param("eps"))
        if not self.tau > 0:
            raise ConfigError("gated_linear_attention: tau must be > 0")
        self.query_scale = float(self.params.get("query_scale", self.dk ** -0.5))
        rank = self.params.get("decay_rank")
        self.rank = int(rank) if rank is not None else None
        self.gate = self.params.get("gate", "silu")
        if self.gate not in kernels.GATE_ACTS:
            raise ConfigError(f"gated_linear_attention: unknown gate '{self.gate}' (known: {sorted(kernels.GATE_ACTS)})")
        self.names = self._names(self.ROLES)

    def state_need(self):
        return StateNeed((self.heads, self.dv, self.dk), "float32")      # [head][value column][key channel]

    def weight_decls(self):
        nk, nv, h, nm = self.heads * self.dk, self.heads * self.dv, self.hidden, self.names
        return [WeightDecl(nm["q"], (nk, h)), WeightDecl(nm["k"], (nk, h)), WeightDecl(nm["v"], (nv, h)),
                WeightDecl(nm["g"], (nv, h)), WeightDecl(nm["a1"], (self.rank, h)), WeightDecl(nm["a2"], (nk, self.rank)),
                WeightDecl(nm["a2_bias"], (nk,), "norm"), WeightDecl(nm["norm"], (self.dv,), "gain"),
                WeightDecl(nm["o"], (h, nv))]

    def load(self, weights):
        nm, f32 = self.names, torch.float32
        self.rank = weights[nm["a1"]].shape[0]
        if weights[nm["a2"]].shape[1] != self.rank:
            raise ConfigError(f"gated_linear_attention: {nm['a1']} has {self.rank} rows, {nm['a2']} has "
                              f"{weights[nm['a2']].shape[1]} columns")
        self.w_in, self.off = self._pack(weights, ("q", "k", "v", "g", "a1"))
        self.w2t = weights[nm["a2"]].to(f32).t().contiguous()            # [rank, heads * dim]: channels side by side
        self.a2_bias = weights[nm["a2_bias"]].to(f32).contiguous()
        self.norm_w = weights[nm["norm"]].to(f32).repeat(self.heads).contiguous()      # the heads share it
        self.w_o = weights[nm["o"]].to(self.ctx.compute_dtype).contiguous()

    def decode_bytes(self, lens) -> int:
        weights = (self.w_in.numel() + self.w_o.numel()) * _el(self.ctx) + 4 * self.w2t.numel()
        return weights + len(lens) * 2 * 4 * self.heads * self.dk * self.dv      # the state, read and written

    def prefill_flops(self, lens) -> int:
        T = sum(lens)
        return 2 * T * (self.w_in.numel() + self.w_o.numel() + self.w2t.numel()) + T * self.heads * 5 * self.dk * self.dv

    def _chunk(self, batch) -> int:
        """Tokens of a chunk for this prefill step's scan, or 0: the sequences as they are.  The token-by-token scan
        has a block a (sequence, head, 32 value columns); while those leave half the SMs without one, the sequences
        are cut into so many chunks that there are about four blocks an SM, of at least ``kernels.SCAN_CHUNK`` tokens
        (a power of two of them), if that leaves the longest sequence two chunks at least.  (With a block an SM the
        scan already runs near what an SM does with four: chunks then only add the join; measured at 32 heads of 128.)"""
        if not bool(self.params.get("chunked_scan", True)):
            return 0
        sms = kernels.sm_count()
        blocks = batch.n_seqs * self.heads * -(-self.dv // 32)
        if 2 * blocks > sms:
            return 0
        want = -(-4 * sms // blocks)
        chunk = kernels.SCAN_CHUNK
        while chunk * want < batch.max_len and chunk < 4096:
            chunk *= 2
        return chunk if batch.max_len >= 2 * chunk else 0

    def forward(self, x, batch, view):
        T, off, f32 = x.shape[0], self.off, torch.float32
        nk, nv = self.heads * self.dk, self.heads * self.dv
        proj = linear(x, self.w_in, out_dtype=f32)
        alpha = torch.empty(T, nk, dtype=f32, device=x.device)
        kernels.channel_decay(alpha, proj, off["a1"], self.w2t, self.a2_bias, self.tau)
        o = torch.empty(T, nv, dtype=f32, device=x.device)
        q, k, v = (proj[:, off[n]: off[n] + w] for n, w in (("q", nk), ("k", nk), ("v", nv)))
        # few long prompts: their tokens one after the other leave most of the GPU idle (a block a head and tile of
        # value columns); cut into chunks that are scanned side by side and joined, the same sums fill it
        chunk = self._chunk(batch) if batch.is_prefill else 0
        if chunk:
            kernels.state_scan_chunked(o, q, k, v, alpha, view.state, batch, self.heads, self.dk, self.dv, chunk=chunk)
        else:
            kernels.state_scan("channel", o, q, k, v, view.state, batch, self.heads, self.dk, self.dv, w=alpha)
        y = torch.empty(T, nv, dtype=x.dtype, device=x.device)
        kernels.gated_group_norm(y, o, self.norm_w, proj[:, off["g"]: off["g"] + nv], self.dv, self.eps,
                                 gate_act=self.gate, in_scale=self.query_scale)
        return linear_split(y, self.w_o, wide=self.wide)
