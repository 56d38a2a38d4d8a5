"""Rotary position encoding with rotate-half pairing.

half = rot/2; f_j = 1/theta^(j/half); angle = (float)pos * f_j; dimension j pairs with
j + half (reference: st.c:8937-8948 for the frequencies, st.c:8963-8989 for the pairing).  The
frequencies are made once on the host in float32 and kept on the device; angles, cos and sin
are computed in float32 inside the kernel that rotates (`ops.attn_prepare`).  ``rotary_dim``
below the head size rotates only the first dimensions of a head; Qwen3 rotates all.  A
`FrequencyScaling` stretches the long wavelengths.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from .base import PositionEncoding, Rotation


@dataclass(frozen=True)
class FrequencyScaling:
    """Stretching of a rotary encoding's long wavelengths for contexts beyond the ``original`` one, by
    bands of the wavelength l = 2 pi / f: l < original / high keeps f; l > original / low takes
    f / factor; between them f is blended, (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low)."""
    factor: float
    low: float
    high: float
    original: float

    def apply(self, freq: np.ndarray) -> np.ndarray:
        f = np.asarray(freq, dtype=np.float64)
        wave = 2.0 * math.pi / f
        s = (self.original / wave - self.low) / (self.high - self.low)
        blended = (1.0 - s) * f / self.factor + s * f
        return np.where(wave < self.original / self.high, f, np.where(wave > self.original / self.low, f / self.factor, blended))


@dataclass(frozen=True)
class RampScaling:
    """Stretching of a rotary encoding by a ramp over the pair index (the scheme published as YaRN): with
    where(t) = dims ln(original / (2 pi t)) / (2 ln base) the pair index whose wavelength fits t times into the original
    context, lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1) and ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1), pair i turns with f_i / factor * ramp_i + f_i (1 - ramp_i).  `magnitude` is the factor the
    scheme puts on cos and sin, 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float
    dims: int
    base: float

    def apply(self, freq: np.ndarray) -> np.ndarray:
        f = np.asarray(freq, dtype=np.float64)

        def where(turns: float) -> float:
            return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
        lo = max(math.floor(where(self.fast)), 0)
        hi = min(math.ceil(where(self.slow)), self.dims - 1)
        ramp = np.clip((np.arange(f.shape[0], dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp)

    @property
    def magnitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0


class RotaryHalf(PositionEncoding):
    graph_safe = True

    pairing = "half"

    def __init__(self, head_dim: int, theta: float, device, rotary_dim: Optional[int] = None, scale: float = 1.0,
                 scaling: Optional[FrequencyScaling] = None):
        rot = head_dim if rotary_dim is None else rotary_dim
        if rot % 2 or rot <= 0 or rot > head_dim:
            raise ValueError(f"rotary size {rot} must be even and at most the head size {head_dim}")
        self.rotary_dim = rot
        self.theta = float(theta)
        self.scale = float(scale)
        self.scaling = scaling
        half = rot // 2
        if scaling is None:
            j = np.arange(half, dtype=np.float32)
            inv = (np.float32(1.0) / np.power(np.float32(theta), j / np.float32(half), dtype=np.float32))
        else:       # the bands are decided on the frequencies in float64; the kernel gets them rounded to float32
            inv = scaling.apply(np.power(float(theta), -np.arange(half, dtype=np.float64) / half))
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(device)

    def rotary(self) -> Rotation:
        return Rotation(self.inv_freq, self.rotary_dim, self.pairing, self.scale)


class RotaryInterleaved(RotaryHalf):
    """The same angles with adjacent pairing: dimension 2j turns with 2j + 1.  No model of the
    reference uses it on this path (its history notes the pairing as a past fault,
    st.c:16478-16483); checkpoints of other families store their heads this way."""

    pairing = "interleaved"


class NoPositionEncoding(PositionEncoding):
    """A mixer that sees no positions (causality alone orders the tokens)."""


class SinusoidalPositions(PositionEncoding):
    """An absolute encoding added to the embedded tokens: entry 2i of position p is
    sin(p * base^(-2i/width)), entry 2i + 1 the cosine of the same angle.  The frequencies are
    made once on the host (in float64, rounded to float32); the angle and its sine and cosine
    are float32 in the kernel.  Mixers get no rotation from it."""

    graph_safe = True

    def __init__(self, width: int, device, base: float = 10000.0):
        self.width, self.base = width, float(base)
        i = np.arange((width + 1) // 2, dtype=np.float64)
        self.freq = torch.from_numpy(np.power(self.base, -2.0 * i / width).astype(np.float32)).to(device)

    def add_to_embedding(self, x: torch.Tensor, batch) -> None:
        from ..csrc import ops
        ops.add_sinusoid(x, batch.positions, self.freq)
