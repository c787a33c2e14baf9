"""Rotary position encoding with half-split pairing: dimension i turns with
dimension i + head_dim/2 by the angle pos * theta^(-i / (head_dim/2))
(reference: src/kernels/mod.rs:572-608).  The part owns the table of inverse
frequencies and names the pairing; the mixer's kernel applies the rotation where
it reads q and k, with angle, sine and cosine in 32-bit."""
from __future__ import annotations

import math

import torch

from ..config.spec import PartSpec
from .registry import register_position
from .runtime import Runtime

STYLE_HALF_SPLIT = 0
STYLE_INTERLEAVED = 1


@register_position("rope_half_split")
class RotaryHalfSplit:
    """Parameters: `head_dim`, `theta`; optionally `scaling` = {factor, low, high, original}, which
    stretches the frequencies band by band: with wavelength l = 2 pi / f, f stays where l < original / high,
    becomes f / factor where l > original / low, and in between is the blend (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low).  Interface of every rotary position part: `inv_freq`
    ([head_dim/2] float32 on the device) and `style`."""
    style = STYLE_HALF_SPLIT

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.inv_freq = self.frequencies(self.head_dim, self.theta, spec.params.get("scaling")) \
            .to(torch.float32).to(rt.device)

    @staticmethod
    def frequencies(head_dim: int, theta: float, scaling=None) -> torch.Tensor:
        """The table in 64-bit on the host (rounded to 32-bit once, where it is stored)."""
        half = head_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), i / half)
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / inv
            s = (original / wave - low) / (high - low)
            blend = (1.0 - s) * inv / factor + s * inv
            inv = torch.where(wave < original / high, inv, torch.where(wave > original / low, inv / factor, blend))
        return inv


@register_position("rope_interleaved")
class RotaryInterleaved(RotaryHalfSplit):
    """The same frequencies with neighbouring pairs: dimension 2i turns with dimension 2i + 1."""
    style = STYLE_INTERLEAVED
