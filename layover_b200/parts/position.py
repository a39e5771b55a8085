"""Position encodings that a mixer applies to its queries and keys."""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import Part, register_position


@register_position("rotary_half")
class RotaryHalf(Part):
    """Rotary embedding over the whole head, pairing lane i with lane i + dim/2.

    inv_freq[i] = theta^(-2i/dim) in 32-bit (layover/model.py:185); angle = position * inv_freq;
    x' = x cos + rotate_half(x) sin (layover/model.py:100-102,127-128). The frequencies are made once
    at build time; `tables(batch)` makes the step's cos/sin table [T, 2, dim/2] in 32-bit once per
    step (every layer with the same head size and theta shares it, as the reference computes its
    tables once per call, layover/model.py:220-221); the rotation itself runs inside the mixer's
    fused kernel.

    params: dim (the head's size), theta; optional `rotated` (only the first `rotated` channels of a head
    turn, channel i paired with channel i + rotated/2, frequencies theta^(-2i/rotated); default: the whole
    head), `linear_factor` (every frequency is divided by it: positions are read on a coarser scale;
    default 1) and `band_scaling` = {factor, low, high, original}: frequencies are rescaled by wavelength
    l = 2 pi / f: kept where l < original / high, divided by `factor` where l > original / low, and in between
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low). With any of them the frequencies
    are made in float64 and rounded once to 32-bit."""

    pairing = "half"

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.require("dim", "theta")
        self.dim, self.theta = int(params["dim"]), float(params["theta"])
        self.rotated = int(params.get("rotated") or self.dim)
        self.linear_factor = float(params.get("linear_factor") or 1.0)
        if self.rotated % 2 or not 0 < self.rotated <= self.dim:
            raise ValueError(f"rotary_half rotates an even number of channels up to the head size, got {self.rotated} of {self.dim}")
        if not self.linear_factor > 0:
            raise ValueError("rotary_half: linear_factor must be positive")
        band = params.get("band_scaling")
        self.band = None
        if band:
            self.band = tuple(float(band[k]) for k in ("factor", "low", "high", "original"))
            if not (self.band[0] > 0 and self.band[2] > self.band[1] >= 0 and self.band[3] > 0):
                raise ValueError(f"rotary: band_scaling needs factor > 0, high > low >= 0 and original > 0, got {band!r}")
        self._table = None

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        if self.rotated == self.dim and self.linear_factor == 1.0 and self.band is None and self.pairing == "half":
            exponent = torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim
            self._table = (1.0 / (self.theta ** exponent)).to(runtime.device).contiguous()
        else:
            exponent = torch.arange(0, self.rotated, 2, dtype=torch.float64) / self.rotated
            freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -exponent) / self.linear_factor
            if self.band is not None:
                factor, low, high, original = self.band
                wave = 2.0 * math.pi / freq
                blend = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
                mixed = (1.0 - blend) * freq / factor + blend * freq
                freq = torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mixed))
            self._table = freq.to(torch.float32).to(runtime.device).contiguous()

    def kernel_libraries(self, dtype):
        return ("elementwise",)

    def inv_freq(self) -> torch.Tensor:
        return self._table

    def tables(self, batch) -> torch.Tensor | None:
        """The step's cos/sin table for the fused kernel; parts that cannot be fused return None."""
        key = ("rotary", self.theta, self.rotated, self.linear_factor, self.band)    # the pairing is the reader's business
        table = batch.shared.get(key)
        if table is None:
            table = torch.empty((batch.n_tokens, 2, self.rotated // 2), dtype=torch.float32, device=self._table.device)
            ops.rope_table(batch.positions, self._table, table)
            batch.shared[key] = table
        return table

    def apply(self, q, k, positions):  # only reached when a mixer cannot fuse the rotation
        raise NotImplementedError("the rotation runs inside the mixer's fused kernel")


@register_position("rotary_pairs")
class RotaryPairs(RotaryHalf):
    """The same rotation with neighbouring channels as pairs: channel 2i turns together with channel 2i + 1
    (i < rotated / 2) by angle position * theta^(-2i / rotated). The step's table has the same form as
    `rotary_half`'s, [T, 2, rotated / 2]; the pairing is applied by the kernel of the mixer that reads it
    (`pairing`). params as `rotary_half`."""

    pairing = "neighbours"
