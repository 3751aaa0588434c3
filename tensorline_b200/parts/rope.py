"""Rotary position encoding, rotate-half pairing (tensorline/fused.py:34-51, :83-85).

tzar-beep/Tensorline takes the cos/sin table from an installed package
(tensorline/paged.py:241-242); the table here is the standard one: inv_freq[i] = theta^(-2i/rot),
i in [0, rot/2), held in float32; the angle pos * inv_freq[i] and its cosine and sine are
computed in float32 inside the kernel that also writes k and v to their pages.  `rotary_dim`
smaller than the head size leaves the remaining dimensions unrotated.  `scaling` {factor, low, high, original} stretches
the long wavelengths (Llama 3.1's rule): with l = 2 pi / f, f stays where l < original / high, becomes f / factor where
l > original / low, and in between is (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
"""
from __future__ import annotations

import math

import torch

from .base import Part, Rotary, Runtime, register_position_encoding


@register_position_encoding("rotary_half")
class RotaryHalf(Part):
    graph_capturable = True
    pairing = "half"

    def __init__(self, rt: Runtime, head_dim: int, theta: float, rotary_dim: int | None = None, scaling: dict | None = None):
        super().__init__(rt)
        rot = head_dim if rotary_dim is None else rotary_dim
        if rot % 2 or rot > head_dim or rot < 0:
            raise ValueError(f"rotary_dim {rot} must be even and at most head_dim {head_dim}")
        self.rot = rot
        i = torch.arange(0, rot, 2, dtype=torch.float64)
        f = float(theta) ** (-i / rot)
        if scaling is not None:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            if not (factor > 0 and high > low > 0 and original > 0):
                raise ValueError(f"frequency scaling {scaling!r}: factor, original > 0 and high > low > 0")
            wavelength = 2.0 * math.pi / f
            s = (original / wavelength - low) / (high - low)
            blended = (1.0 - s) * f / factor + s * f
            f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
        self.inv_freq = f.to(torch.float32).to(rt.device)

    def rotary(self):
        return Rotary(self.inv_freq, self.rot, self.pairing)

    def on_embedding(self, x, ctx):
        return None


@register_position_encoding("rotary_interleaved")
class RotaryInterleaved(RotaryHalf):
    """The same table; pair i is dimensions (2i, 2i + 1)."""
    pairing = "interleaved"


@register_position_encoding("none")
class NoPositionEncoding(Part):
    graph_capturable = True

    def __init__(self, rt: Runtime, **_):
        super().__init__(rt)
        self._empty = torch.zeros(0, dtype=torch.float32, device=rt.device)

    def rotary(self):
        return Rotary(self._empty, 0)

    def on_embedding(self, x, ctx):
        return None
