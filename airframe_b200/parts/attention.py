"""Grouped-query attention over the paged cache, with score scale, softcap
and an optional window.

score = softcap(q.k * scale), softmax over the visible keys in 32 bits, times
v; query head h reads key/value head h // (heads / kv_heads).  Reference:
``src/backend/bindless/sh_layer_v1.wgsl:662-754`` (scale ``:726``, cap
``:727-730``, online softmax ``:739-753``, head mapping ``:673,677``), the
projections ``:499-530`` and ``:775-804``.  The reference fixes the scale at
head_dim^-0.5 and has no window; both are parameters here.

Two more options, for designs that have them: ``qk_norm`` (q and k heads are
RMS-normed per head with a weight of head_dim values that all heads share,
before any rotation) and values taken from the raw key projection (no
``v_weight``: v = W_k h, before norm and rotation).  With either, the
projection goes into 32-bit rows and one kernel norms, rotates, packs
[q | k | v] and writes the cache.

More options that go the same way: biases of the q, k and v projections; q and k
divided by their root mean square per head *after* the rotation (no weight); values
of another size than the keys (``value_dim``); a chunked mask (``mask`` = "chunk": a
position sees the earlier positions of its own chunk of ``window`` positions, chunks
counted from position 0) instead of the sliding one; a learned sink per head in the
softmax's denominator; an output gate, one number per head and token (the sigmoid of
a projection of the mixer's input), that multiplies the head's output before the
output projection; and ``qk_norm`` taken over a token's whole q (and whole k)
projection, all heads at once, with weights of that size.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError, PartSpec
from ..weights.loader import WeightDecl
from .base import KVNeed, Mixer, PositionEncoding, build_part, register_part
from .linear import PartialSums, linear, linear_split
from .rope import Rope


@register_part("mixer", "attention")
class Attention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``scale``, ``softcap`` (0 = off), ``window`` (None = all keys), ``position``
    (a PartSpec of category ``position``), ``q_weight``/``k_weight``/``v_weight``/
    ``o_weight`` (tensor names; ``v_weight`` None or absent: the values are the keys as
    projected); optional ``qk_norm``: {``q_weight``, ``k_weight`` (tensor names of head_dim
    values each), ``eps``}; optional ``wide_output`` (default false): the output projection's
    result stays float32 on its way into the residual sum; optional ``value_dim`` (default ``head_dim``);
    optional ``mask`` ("window", the default, or "chunk") that says what ``window`` means; optional ``q_bias``,
    ``k_bias``, ``v_bias`` (tensor names; all or none); ``qk_norm`` may instead be {``after_rotation``: true,
    ``eps``} (no weights: q and k over their root mean square once they are rotated), or carry ``whole``: true
    (the mean square is taken over all heads of the token's q, and of its k, and the two weights hold
    heads x head_dim and kv heads x head_dim values); optional ``gate_weight``
    (tensor name, [heads, hidden]: the output gate) and ``sink_weight`` (tensor name, [heads]);
    optional ``rope_epilogue`` (default false): run the
    q, k, v projection with the rotary encoding and the cache write in its epilogue
    (``kernels.gemm_tc_rope``) where sizes and encoding allow.  Off by default
    because it measures slower than the projection followed by the rotary kernel:
    four epilogue warps a block cannot hide the latency of the table of cosines
    that many blocks of the rotary kernel hide easily (Gemma-2 2B sizes: a
    2,048-token prompt 9.6 ms against 8.3, a decode step at batch 8 1.93 ms against 1.75)."""

    @property
    def graph_safe(self):
        return self.position.graph_safe


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.nq = int(self.param("num_heads"))
        self.nkv = int(self.param("num_kv_heads"))
        self.hd = int(self.param("head_dim"))
        self.scale = float(self.param("scale"))
        self.softcap = float(self.params.get("softcap") or 0.0)
        w = self.params.get("window")
        self.window = int(w) if w else None
        if self.nq % self.nkv:
            raise ConfigError(f"attention: {self.nq} heads are not a multiple of {self.nkv} kv heads")
        pos = self.params.get("position") or PartSpec("none")
        self.position = build_part("position", pos, ctx)
        self.names = [self.param("q_weight"), self.param("k_weight"), self.params.get("v_weight"),
                      self.param("o_weight")]
        self.v_from_k = self.names[2] is None
        self.qk_norm = self.params.get("qk_norm")
        self.norm_after = bool(self.qk_norm and self.qk_norm.get("after_rotation"))
        self.norm_whole = bool(self.qk_norm and self.qk_norm.get("whole"))
        if self.norm_whole and self.norm_after:
            raise ConfigError("attention: 'qk_norm' over the whole projection comes before the rotation")
        if self.qk_norm is not None:
            wanted = ("eps",) if self.norm_after else ("q_weight", "k_weight", "eps")
            missing = [k for k in wanted if k not in self.qk_norm]
            if missing:
                raise ConfigError(f"attention: 'qk_norm' needs {missing}")
        self.dv = int(self.params.get("value_dim") or self.hd)
        self.mask = self.params.get("mask") or "window"
        if self.mask not in kernels.MASKS:
            raise ConfigError(f"attention: unknown mask '{self.mask}' (known: {sorted(kernels.MASKS)})")
        self.bias_names = [self.params.get(k) for k in ("q_bias", "k_bias", "v_bias")]
        if any(self.bias_names) and not (all(self.bias_names[:2]) and (self.v_from_k or self.bias_names[2])):
            raise ConfigError("attention: biases for all of q, k and v, or for none")
        self.gate_name = self.params.get("gate_weight")
        self.sink_name = self.params.get("sink_weight")
        if self.v_from_k and self.dv != self.hd:
            raise ConfigError("attention: values that are the keys have their size")
        # norm, biases, a gate, shared or odd-sized values: the projection is packed by the kernel that norms,
        # rotates and stores, which knows rotations (a rotary encoding or none) and nothing else that rewrites q and k
        self.packs = (self.v_from_k or self.qk_norm is not None or any(self.bias_names) or self.gate_name is not None
                      or self.dv != self.hd)
        if self.packs and not isinstance(self.position, Rope) \
                and type(self.position).encode is not PositionEncoding.encode:
            raise ConfigError(f"attention: qk_norm and shared values go with a rotary encoding or none, "
                              f"not with '{self.position.kind}'")
        # bfloat16 heads of a size the tensor-core attention kernels do not take are padded with zeros up to one they
        # do (96 -> 128), in the packed rows and in the cache, where that costs at most twice the elements: the
        # packing kernel writes the padding, the output projection's weight gets zero columns for it
        self.pad = 0
        big = max(self.hd, self.dv)
        if ctx.compute_dtype == torch.bfloat16 and self.packs and not self.v_from_k:
            fit = next((p for p in kernels.FAST_HEAD_SIZES if p >= big), 0)
            if fit and fit <= 2 * big and (fit != self.hd or fit != self.dv):
                self.pad = fit
        self.q_norm_w = self.k_norm_w = self.bias = self.sinks = None
        self.w_qkv = None
        self.w_o = None
        self.rope_epilogue = False

    def kv_need(self):
        # (a chunk's keys all lie within the last ``window`` positions: the ring of a window serves it)
        if self.pad:
            return KVNeed(self.nkv, self.pad, self.window)
        return KVNeed(self.nkv, self.hd, self.window, None if self.dv == self.hd else self.dv)

    def weight_decls(self):
        q, k, v, o = self.names
        decls = [WeightDecl(q, (self.nq * self.hd, self.hidden)),
                 WeightDecl(k, (self.nkv * self.hd, self.hidden))]
        if v is not None:
            decls.append(WeightDecl(v, (self.nkv * self.dv, self.hidden)))
        decls.append(WeightDecl(o, (self.hidden, self.nq * self.dv)))
        if self.qk_norm is not None and not self.norm_after:
            nq_w, nk_w = (self.nq * self.hd, self.nkv * self.hd) if self.norm_whole else (self.hd, self.hd)
            decls += [WeightDecl(self.qk_norm["q_weight"], (nq_w,), "norm"),
                      WeightDecl(self.qk_norm["k_weight"], (nk_w,), "norm")]
        for name, rows in zip(self.bias_names, (self.nq * self.hd, self.nkv * self.hd, self.nkv * self.dv)):
            if name:
                decls.append(WeightDecl(name, (rows,), "norm"))
        if self.gate_name:
            decls.append(WeightDecl(self.gate_name, (self.nq, self.hidden)))
        if self.sink_name:
            decls.append(WeightDecl(self.sink_name, (self.nq,), "norm"))
        return [*decls, *self.position.weight_decls()]

    def load(self, weights):
        q, k, v, o = self.names
        dt = self.ctx.compute_dtype
        # one matrix product for q, k and v: rows [q heads | k heads | v heads]
        mats = [weights[q], weights[k]] + ([weights[v]] if v is not None else [])
        if self.gate_name:
            mats.append(weights[self.gate_name])        # the gate's logits ride behind [q | k | v] in the same product
        self.w_qkv = torch.cat(mats, dim=0).to(dt).contiguous()
        if any(self.bias_names):
            self.bias = torch.cat([weights[n].to(torch.float32).reshape(-1) for n in self.bias_names if n]).contiguous()
        if self.sink_name:
            self.sinks = weights[self.sink_name].to(torch.float32).contiguous()
        self.w_o = weights[o].to(dt).contiguous()
        if self.pad:
            wide = torch.zeros(self.hidden, self.nq, self.pad, dtype=dt, device=self.w_o.device)
            wide[:, :, : self.dv] = self.w_o.view(self.hidden, self.nq, self.dv)
            self.w_o = wide.view(self.hidden, self.nq * self.pad).contiguous()
        self.position.load(weights)
        if self.qk_norm is not None and not self.norm_after:
            self.q_norm_w = weights[self.qk_norm["q_weight"]].to(torch.float32).contiguous()
            self.k_norm_w = weights[self.qk_norm["k_weight"]].to(torch.float32).contiguous()
        # bfloat16 with a head size and a K that the tensor-core product takes: the rows of every head in the
        # order in which the product's epilogue rotates pairs and writes the cache (used only when the position
        # encoding says, step by step, that it is such a rotation)
        self.rope_epilogue = (bool(self.params.get("rope_epilogue")) and not self.packs and dt == torch.bfloat16 and self.hd % 32 == 0
                              and self.hidden % 8 == 0 and self.w_qkv.is_cuda
                              and self.position.rotates_half_pairs(self.hd))
        if self.rope_epilogue:
            order = kernels.rope_row_order(self.nq + 2 * self.nkv, self.hd, self.w_qkv.device)
            self.w_qkv = self.w_qkv.index_select(0, order).contiguous()
            self.tickets = torch.zeros(4 * ((self.w_qkv.shape[0] + 127) // 128), dtype=torch.int32,
                                       device=self.w_qkv.device)

    def _el(self) -> int:
        return 4 if self.ctx.compute_dtype == torch.float32 else 2

    def decode_bytes(self, lens) -> int:
        weights = (self.w_qkv.numel() + self.w_o.numel()) * self._el()
        kv_row = self.nkv * (2 * self.pad if self.pad else self.hd + self.dv) * self._el()
        return weights + sum(kv_row * self._visible(n - 1) for n in lens)

    def _visible(self, pos: int) -> int:
        """Keys that the token at ``pos`` sees."""
        if not self.window:
            return pos + 1
        return pos % self.window + 1 if self.mask == "chunk" else min(pos + 1, self.window)

    def score_flops(self, lens) -> int:
        """The part of :meth:`prefill_flops` that is scores and their products with v."""
        pairs = 0
        for n in lens:          # visible (query, key) pairs of a causal prompt, with the window where there is one
            w = self.window
            if w and self.mask == "chunk":
                full, rest = divmod(n, w)
                pairs += full * (w * (w + 1) // 2) + rest * (rest + 1) // 2
            else:
                pairs += n * (n + 1) // 2 if not w or n <= w else w * (w + 1) // 2 + (n - w) * w
        return 2 * pairs * self.nq * (self.hd + self.dv)

    def prefill_flops(self, lens) -> int:
        T = sum(lens)
        proj = 2 * T * (self.w_qkv.shape[0] * self.hidden + self.hidden * self.nq * self.dv)
        return proj + self.score_flops(lens)

    def _project_rotate_store(self, x, batch, view):
        """q, k, v rows of the step with positions encoded and k, v stored: the
        product with the rotation and the cache write in its epilogue."""
        nq, nkv, hd = self.nq, self.nkv, self.hd
        table = self.position.rotary_table(batch, hd)
        M, N = x.shape[0], self.w_qkv.shape[0]
        rows = kc = vc = None
        if view.writes:
            kv = view.kv
            key = ("kv_rows", kv.page_table.data_ptr(), kv.ring_rows, nkv)
            if key not in batch.aux:
                batch.aux[key] = kernels.kv_rows(batch, kv, nkv)
            rows, kc, vc = batch.aux[key], kv.k, kv.v
        qkv = torch.empty(M, N, dtype=x.dtype, device=x.device)
        splits = kernels.gemm_tc_splits(M, N, x.shape[1]) if M <= 64 else 1
        kernels.gemm_tc_rope(qkv, x, self.w_qkv, table, nq, nkv, hd, rows, kc, vc, splits=splits,
                             tickets=self.tickets)
        return qkv

    def _project_norm_pack(self, x, batch, view):
        """The projection in 32-bit rows; q and k heads normed and rotated, the values taken
        (from the raw key projection, or their own heads), all packed and the cache written: one kernel."""
        nq, nkv, hd = self.nq, self.nkv, self.hd
        proj = linear(x, self.w_qkv, out_dtype=torch.float32)
        width = (nq + 2 * nkv) * self.pad if self.pad else (nq + nkv) * hd + nkv * self.dv
        qkv = torch.empty(x.shape[0], width, dtype=x.dtype, device=x.device)
        rope = self.position if isinstance(self.position, Rope) else None
        if rope is not None and rope.rotary_dim > hd:
            raise ConfigError(f"rope: rotary_dim {rope.rotary_dim} exceeds head_dim {hd}")
        kernels.qk_norm_rope_store(
            qkv, proj, batch, nq, nkv, hd,
            rope.inv_freq if rope is not None else kernels.no_frequencies(x.device),
            rope.rotary_dim if rope is not None else 0, rope.pairing if rope is not None else "half",
            q_weight=self.q_norm_w, k_weight=self.k_norm_w,
            eps=float(self.qk_norm["eps"]) if self.qk_norm is not None else 0.0,
            v_from_k=self.v_from_k, kv=view.kv if view.writes else None, bias=self.bias,
            norm_after=self.norm_after, magnitude=rope.magnitude if rope is not None else 1.0, dv=self.dv,
            pitch=self.pad, whole_norm=self.norm_whole,
            table=rope.precise_table(batch) if rope is not None else None)
        gate = None
        if self.gate_name:
            at = (nq + nkv) * hd + (0 if self.v_from_k else nkv * self.dv)
            gate = proj[:, at: at + nq]
        return qkv, gate

    def forward(self, x, batch, view):
        nq, nkv, hd = self.nq, self.nkv, self.hd
        kv = view.kv
        gate = None
        if self.packs:
            qkv, gate = self._project_norm_pack(x, batch, view)
        elif self.rope_epilogue:
            qkv = self._project_rotate_store(x, batch, view)
        else:
            qkv = linear_split(x, self.w_qkv)
            parts = None
            if isinstance(qkv, PartialSums):
                parts = qkv.parts
                qkv = torch.empty(x.shape[0], (nq + 2 * nkv) * hd, dtype=x.dtype, device=x.device)
            # positions into q and k, then k and v into the cache: the store is this mixer's; an encoding
            # that can do both in one kernel says so
            if not view.writes:
                self.position.encode(qkv, batch, nq, nkv, hd, parts=parts)
            elif not self.position.encode_and_store(qkv, batch, nq, nkv, hd, kv, parts=parts):
                self.position.encode(qkv, batch, nq, nkv, hd, parts=parts)
                kernels.store_kv(qkv, batch, nq, nkv, hd, kv)
        slopes = self.position.score_slopes(nq)
        dv = self.dv
        if self.pad:                 # (from here on the heads are what the packing kernel made of them)
            hd = dv = self.pad
        q = qkv[:, : nq * hd]
        k = qkv[:, nq * hd: (nq + nkv) * hd]
        v = qkv[:, (nq + nkv) * hd:]
        ctx = torch.empty(x.shape[0], nq * dv, dtype=x.dtype, device=x.device)
        window = self.window or 0
        more = {"dv": dv, "mask": self.mask, "sinks": self.sinks, "gate": gate}
        if batch.is_prefill:
            if not view.writes:
                k, v = batch.step_kv[view.cache_id]
            elif view.keep_step_kv:
                batch.step_kv[view.cache_id] = (k.clone(), v.clone())
            kernels.attn_prefill(ctx, q, k, v, batch, nq, nkv, hd, self.scale, self.softcap, window, slopes, **more)
        else:
            kernels.attn_decode(ctx, q, kv, batch, nq, nkv, hd, self.scale, self.softcap, window, slopes, **more)
        return linear_split(ctx, self.w_o, wide=bool(self.params.get("wide_output", False)))
