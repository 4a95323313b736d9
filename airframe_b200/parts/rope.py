"""Rotary position encoding, applied to q and k before the cache write so
that cached keys are final (a ring of rows then works with plain dot products).

angle = position * theta^(-2p / rotary_dim), computed in 32 bits from a table
of inverse frequencies made in 64 bits.  Reference: ``theta_p`` of
``src/backend/bindless/preflight.rs:87-90``; rotation
``src/ops/reference/rope.rs:156-196`` (absolute) and
``src/backend/bindless/sh_layer_v1.wgsl:706-725`` (relative, at score time).
The reference pairs adjacent elements (GGUF row order); ``pairing`` selects
``half`` (element i with i + rotary_dim/2, Hugging Face row order) or ``adjacent``.

``scaling`` stretches the context a model was trained for: with
turn(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turn(fast)), 0) and
hi = min(ceil(turn(slow)), rotary_dim - 1), pair p gets the ramp r = clamp((p - lo) / max(hi - lo, 0.001), 0, 1) and
the frequency f_p / factor * r + f_p * (1 - r): fast pairs keep their frequency, slow ones are
divided by ``factor``.  Cosines and sines are then multiplied by ``magnitude`` = 0.1 ln(factor) + 1.

``scaling`` with ``kind`` = "wavelength" ({factor, low, high, original}) decides pair by pair from the
wavelength l = 2 pi / f: l < original / high keeps f; l > original / low takes f / factor; between the two,
with s = (original / l - low) / (high - low), the frequency is (1 - s) f / factor + s f.  No magnitude.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.base import ConfigError
from .base import PositionEncoding, register_part


@register_part("position", "rope")
class Rope(PositionEncoding):
    """Parameters: ``theta``, ``rotary_dim``, ``pairing``; optional ``scaling``: {``factor``, ``original``,
    ``fast``, ``slow``}, or {``kind``: "wavelength", ``factor``, ``low``, ``high``, ``original``}; optional
    ``precise_angles`` (default false): a mixer that packs its projection takes the cosines and sines from a
    table of the step that is made from 64-bit frequencies with 64-bit angles (once per step for all layers)."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.theta = float(self.param("theta"))
        self.rotary_dim = int(self.param("rotary_dim"))
        self.pairing = self.param("pairing")
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} must be even")
        if self.pairing not in kernels.PAIRINGS:
            raise ConfigError(f"rope: unknown pairing '{self.pairing}'")
        p = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * p / max(self.rotary_dim, 1))
        self.magnitude = 1.0
        sc = self.params.get("scaling")
        if sc and sc.get("kind", "ramp") not in ("ramp", "wavelength"):
            raise ConfigError(f"rope: unknown kind of 'scaling' '{sc.get('kind')}' (known: ramp, wavelength)")
        if sc and sc.get("kind") == "wavelength":
            missing = [k for k in ("factor", "low", "high", "original") if k not in sc]
            if missing:
                raise ConfigError(f"rope: 'scaling' needs {missing}")
            factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            if not (factor > 0 and original > 0 and low > 0 and high > low):
                raise ConfigError("rope: 'scaling' by wavelength needs positive numbers and high > low")
            wave = 2.0 * math.pi / inv
            s = (original / wave - low) / (high - low)
            mixed = (1.0 - s) * inv / factor + s * inv
            inv = torch.where(wave < original / high, inv, torch.where(wave > original / low, inv / factor, mixed))
        elif sc:
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in sc]
            if missing:
                raise ConfigError(f"rope: 'scaling' needs {missing}")
            factor, original = float(sc["factor"]), float(sc["original"])
            if not (factor > 0 and original > 0 and float(sc["fast"]) > 0 and float(sc["slow"]) > 0 and self.theta > 1):
                raise ConfigError("rope: 'scaling' needs positive numbers and theta > 1")

            def turn(t):
                return self.rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turn(float(sc["fast"]))), 0)
            hi = min(math.ceil(turn(float(sc["slow"]))), self.rotary_dim - 1)
            ramp = ((p - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            inv = inv / factor * ramp + inv * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self._inv_freq_host = inv.to(torch.float32)
        self._inv_freq64_host = inv
        self.precise = bool(self.params.get("precise_angles", False))
        self._table_key = ("rope_table64", inv.numpy().tobytes())
        self.inv_freq = self.inv_freq64 = None

    def load(self, weights):
        self.inv_freq = self._inv_freq_host.to(self.ctx.device)
        if self.precise:
            self.inv_freq64 = self._inv_freq64_host.to(self.ctx.device)

    def precise_table(self, batch):
        """None, or with ``precise_angles`` float32 [T, rotary_dim / 2, 2] of (cos, sin) from 64-bit angles,
        made once per pass (kept in ``batch.aux``)."""
        if not self.precise or self.rotary_dim == 0:
            return None
        key = self._table_key           # (by the frequencies' values: layers that rotate alike share the table)
        if key not in batch.aux:
            batch.aux[key] = kernels.rope_table_precise(batch.positions, self.inv_freq64)
        return batch.aux[key]

    def rotates_half_pairs(self, hd):
        return self.pairing == "half" and self.rotary_dim == hd and self.magnitude == 1.0

    def _plain_only(self):
        if self.magnitude != 1.0:
            raise ConfigError("rope: stretched frequencies with a magnitude go through the mixer's packing kernel "
                              "(kernels.qk_norm_rope_store), which this path is not")

    def rotary_table(self, batch, hd):
        key = ("rope_table", self.theta, self.rotary_dim, self.inv_freq.data_ptr())
        if key not in batch.aux:
            batch.aux[key] = kernels.rope_table(batch.positions, self.inv_freq)
        return batch.aux[key]

    def encode(self, qkv, batch, nq, nkv, hd, parts=None):
        self._plain_only()
        if self.rotary_dim > hd:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} exceeds head_dim {hd}")
        kernels.rope_cache_write(qkv, batch.positions, self.inv_freq, nq, nkv, hd, self.rotary_dim,
                                 self.pairing, parts=parts)

    def encode_and_store(self, qkv, batch, nq, nkv, hd, kv, parts=None) -> bool:
        """The rotation and the mixer's cache store as one kernel (the rotated
        k rows are what the cache keeps)."""
        self._plain_only()
        if self.rotary_dim > hd:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} exceeds head_dim {hd}")
        # many rows (a prompt): the cosines and sines come from the step's table, made once for all layers
        table = None
        if (qkv.shape[0] >= kernels.ROPE_TABLE_ROWS and parts is None and qkv.dtype == torch.bfloat16
                and self.rotates_half_pairs(hd)):
            table = self.rotary_table(batch, hd)
        kernels.rope_cache_write(qkv, batch.positions, self.inv_freq, nq, nkv, hd, self.rotary_dim,
                                 self.pairing, seq_of_token=batch.seq_of_token, slots=batch.slots,
                                 len_after=batch.len_after, kcache=kv.k, vcache=kv.v,
                                 page_table=kv.page_table, ring_rows=kv.ring_rows, parts=parts, table=table)
        return True


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No encoding (the base class's behaviour under a name)."""
    graph_safe = True
