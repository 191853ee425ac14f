"""Position encodings.  Rotary: cos/sin tables in 32-bit, rotate-half pairing.

Tables follow the reference's order of operations in float32
(src/model/rope.hpp:25-28 base frequency, :159-188 YaRN blend, :191-217 fill):
    freq_i  = powf(theta, -2 i / D)
    angle   = (float) pos * freq_i
    cos/sin = cosf / sinf (angle) [* attention factor under YaRN]
indexed [pos, i], i < D / 2.  The mixer's kernel pairs (i, i + rot_dim / 2).

Another position encoding provides the same two things: `prepare` (build what
its kernel reads) and the attributes the mixer hands to the kernel
(`cos`, `sin`, both None for "no rotation").
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .base import Part


def power_frequencies(base: float, dims: int) -> np.ndarray:
    """f_i = base^(-2i / dims), i < dims / 2, in double precision."""
    i = np.arange(dims // 2, dtype=np.float64)
    return np.power(np.float64(base), -2.0 * i / max(dims, 1))


def blended_frequencies(base: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """Frequencies for contexts longer than the `original` one a model was made for, and the factor on cosines and
    sines that goes with them: pair i keeps f_i where it turns often within the original context and takes f_i / factor
    where it turns rarely, with a linear ramp over the pair index in between.  With n(t) = dims ln(original / (2 pi t)) /
    (2 ln base), the pair that makes t turns in `original` positions, the ramp runs from lo = max(floor(n(fast)), 0) to
    hi = min(ceil(n(slow)), dims - 1): ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), and the frequency is
    f_i / factor * ramp_i + f_i (1 - ramp_i).  The factor on cosines and sines is 0.1 ln(factor) + 1.
    Returns (float64 frequencies [dims / 2], magnitude); the caller rounds once to 32-bit."""
    f = power_frequencies(base, dims)

    def pair_turning(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_turning(fast)), 0)
    hi = min(math.ceil(pair_turning(slow)), dims - 1)
    ramp = np.clip((np.arange(dims // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def banded_frequencies(base: float, dims: int, factor: float, low: float, high: float, original: float) -> np.ndarray:
    """Frequencies changed by wavelength for contexts longer than the `original` one: with l = 2 pi / f_i, a pair keeps f_i
    where l < original / high, takes f_i / factor where l > original / low, and in between, with s = (original / l - low) /
    (high - low), takes (1 - s) f_i / factor + s f_i.  Returns float64 [dims / 2]; the caller rounds once to 32-bit."""
    f = power_frequencies(base, dims)
    wavelength = 2.0 * math.pi / f
    s = (original / wavelength - low) / (high - low)
    out = (1.0 - s) * f / factor + s * f
    out = np.where(wavelength < original / high, f, out)
    return np.where(wavelength > original / low, f / factor, out)


class NoPositionEncoding(Part):
    cos = None
    sin = None
    rot_dim = 0


class RotaryEmbedding(Part):
    def __init__(self, head_dim: int, theta: float, rot_dim: Optional[int] = None, yarn=None,
                 max_positions: Optional[int] = None):
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim if rot_dim is not None else head_dim)
        if self.rot_dim % 2 or self.rot_dim > self.head_dim or self.rot_dim <= 0:
            raise ValueError("the rotated width must be even, positive and at most the head width")
        self.theta = float(theta)
        self.yarn = yarn
        self.max_positions = max_positions
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def frequencies(self) -> np.ndarray:
        dim, half = self.rot_dim, self.rot_dim // 2
        i = np.arange(half, dtype=np.float32)
        theta = np.float32(self.theta)
        if self.yarn is None:
            return np.power(theta, np.float32(-2.0) * i / np.float32(dim)).astype(np.float32)
        y = self.yarn

        def correction(rotations: float) -> float:
            return dim * math.log(y.original_max_position_embeddings / (rotations * 2 * math.pi)) / (2 * math.log(self.theta))

        low = max(math.floor(correction(y.beta_fast)), 0.0)
        high = min(math.ceil(correction(y.beta_slow)), float(dim - 1))
        if low == high:
            high += 0.001
        power = np.power(theta, (np.float32(2.0) * i) / np.float32(dim)).astype(np.float32)
        extra = np.float32(1.0) / power
        inter = np.float32(1.0) / (np.float32(y.factor) * power)
        ramp = np.clip((i - np.float32(low)) / np.float32(high - low), np.float32(0), np.float32(1)).astype(np.float32)
        extrapolate = np.float32(1.0) - ramp
        return (inter * (np.float32(1.0) - extrapolate) + extra * extrapolate).astype(np.float32)

    def tables(self, positions: int):
        freq = self.frequencies()
        pos = np.arange(positions, dtype=np.float32)[:, None]
        angle = (pos * freq[None, :]).astype(np.float32)
        cos, sin = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
        if self.yarn is not None:
            scale = np.float32(self.yarn.attention_factor)
            cos, sin = cos * scale, sin * scale
        return cos, sin

    def prepare(self, max_positions: int, device) -> None:
        n = max_positions if self.max_positions is None else min(max_positions, self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n and self.cos.device == torch.device(device):
            return
        cos, sin = self.tables(n)
        self.cos = torch.from_numpy(cos).to(device).contiguous()
        self.sin = torch.from_numpy(sin).to(device).contiguous()
