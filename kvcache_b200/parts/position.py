"""Position encodings.  The one this architecture uses rotates queries and keys
(rotate-half pairing; reference: src/qwen_kernels.cu:63-78, per-row positions :253-264)."""
from __future__ import annotations

import math
from typing import Mapping, Optional

import numpy as np
import torch

from .base import PositionEncoding, Rotation


class RampScaling:
    """Stretches the slow dimension pairs of a rotation for contexts longer than the `original` one.

    Pair t turns `original * f_t / (2 pi)` times over the original context.  With
    pair_of(turns) = dims * ln(original / (2 pi turns)) / (2 ln base), lo = max(floor(pair_of(fast)), 0) and
    hi = min(ceil(pair_of(slow)), dims - 1), the ramp r_t = clamp((t - lo) / max(hi - lo, 0.001), 0, 1) blends the
    frequency: f_t / factor * r_t + f_t * (1 - r_t) - pairs that turn often keep theirs, pairs that turn seldom are
    slowed by `factor`.  cos and sin are both multiplied by 0.1 ln(factor) + 1.
    """

    def __init__(self, factor: float, original: float, fast: float, slow: float):
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)

    def key(self) -> tuple:
        return (self.factor, self.original, self.fast, self.slow)

    def blend(self, freq: np.ndarray, dims: int, base: float) -> np.ndarray:
        pair_of = lambda turns: dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(pair_of(self.fast)), 0)
        hi = min(math.ceil(pair_of(self.slow)), dims - 1)
        ramp = np.clip((np.arange(len(freq), dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / self.factor * ramp + freq * (1.0 - ramp)

    def gain(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0


class WavelengthScaling:
    """Slows the pairs of a rotation by their wavelength l = 2 pi / f against the `original` context: pairs with
    l < original / high keep f, pairs with l > original / low turn at f / factor, and between the two the frequency is
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  cos and sin keep their size."""

    def __init__(self, factor: float, low: float, high: float, original: float):
        self.factor, self.low, self.high, self.original = float(factor), float(low), float(high), float(original)

    def key(self) -> tuple:
        return (self.factor, self.low, self.high, self.original)

    def blend(self, freq: np.ndarray, dims: int, base: float) -> np.ndarray:
        wavelength = 2.0 * math.pi / freq
        s = (self.original / wavelength - self.low) / (self.high - self.low)
        mixed = (1.0 - s) * freq / self.factor + s * freq
        return np.where(wavelength < self.original / self.high, freq,
                        np.where(wavelength > self.original / self.low, freq / self.factor, mixed))

    def gain(self) -> float:
        return 1.0


class RotaryHalf(PositionEncoding):
    """Pairs dimension t with t + rotary_dim/2; angle = pos * theta^(-2t / rotary_dim).

    The cos/sin tables for positions 0..max_positions-1 are made once on the
    host in double precision and rounded to float32, so the angle of a far
    position carries no accumulated float32 error.
    """

    def __init__(self, rotary_dim: int, theta: float, max_positions: int, scaling=None):
        """`scaling`: None, or an object with `blend(freq, dims, base) -> freq` and `gain()` (`RampScaling`,
        `WavelengthScaling`)."""
        if rotary_dim % 2 != 0 or rotary_dim < 2:
            raise ValueError(f"rotary_dim must be even and positive, got {rotary_dim}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.scaling = scaling
        self._rotation: Optional[Rotation] = None

    def frequencies(self) -> np.ndarray:
        """The angle per position of every dimension pair, in double precision."""
        half = self.rotary_dim // 2
        freq = self.theta ** (-(np.arange(half, dtype=np.float64) * 2.0) / self.rotary_dim)
        return freq if self.scaling is None else self.scaling.blend(freq, self.rotary_dim, self.theta)

    def bind(self, tensors: Mapping[str, torch.Tensor], device: torch.device) -> None:
        if self._rotation is not None and self._rotation.cos.device == torch.device(device):
            return                       # one encoding may serve several mixers: its table is made once
        angles = np.arange(self.max_positions, dtype=np.float64)[:, None] * self.frequencies()[None, :]
        gain = 1.0 if self.scaling is None else self.scaling.gain()
        cos = torch.from_numpy((np.cos(angles) * gain).astype(np.float32)).to(device).contiguous()
        sin = torch.from_numpy((np.sin(angles) * gain).astype(np.float32)).to(device).contiguous()
        self._rotation = Rotation(cos=cos, sin=sin)

    def rotation(self) -> Optional[Rotation]:
        return self._rotation


class NoPositionEncoding(PositionEncoding):
    pass
