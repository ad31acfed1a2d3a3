"""Rotary position encoding: the table of angles, built on the host.

Base frequencies as the reference computes them, ``inv_freq[i] = 1.0f / powf(theta,
(float)(2i) / (float)hd)`` in 32-bit (src/model.cpp:220-225), the angle ``(float)pos *
inv_freq[i]`` and its ``cosf`` / ``sinf`` (src/kernels.cpp:276-279), all through the C
library so that a CPU implementation calling the same functions sees the same bits; the
kernels only read the table.  The ``llama3`` rescaling of the frequencies is not in the
reference (tools/convert.py:59-60 rejects rope_scaling): wavelengths shorter than
``orig / high_freq_factor`` stay, longer than ``orig / low_freq_factor`` are divided by
``factor``, the band between is blended linearly; evaluated in 64-bit from the 32-bit base
value and rounded once.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding

_libm = ctypes.CDLL("libm.so.6")
_libm.powf.restype = ctypes.c_float
_libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
for _n in ("cosf", "sinf"):
    getattr(_libm, _n).restype = ctypes.c_float
    getattr(_libm, _n).argtypes = [ctypes.c_float]


def inverse_frequencies(head_dim: int, theta: float, scaling=None) -> np.ndarray:
    half = head_dim // 2
    theta32 = float(np.float32(theta))
    inv = np.empty(half, dtype=np.float32)
    for i in range(half):
        expo = np.float32(np.float32(2 * i) / np.float32(head_dim))
        inv[i] = np.float32(1.0) / np.float32(_libm.powf(theta32, float(expo)))
    if scaling is None:
        return inv
    lo_wave = scaling.original_max_position_embeddings / scaling.low_freq_factor
    hi_wave = scaling.original_max_position_embeddings / scaling.high_freq_factor
    out = np.empty(half, dtype=np.float32)
    for i in range(half):
        f = float(inv[i])
        wavelen = 2.0 * math.pi / f
        if wavelen < hi_wave:
            v = f
        elif wavelen > lo_wave:
            v = f / scaling.factor
        else:
            smooth = (scaling.original_max_position_embeddings / wavelen - scaling.low_freq_factor) / (
                scaling.high_freq_factor - scaling.low_freq_factor)
            v = (1.0 - smooth) * f / scaling.factor + smooth * f
        out[i] = np.float32(v)
    return out


class RotaryEncoding(PositionEncoding):
    """cos / sin tables [positions, head_dim / 2] in float32, grown on demand."""
    graph_safe = True  # kernels only: a step through this part can be captured


    def __init__(self, head_dim: int, theta: float, scaling=None, positions: int = 0):
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {head_dim}")
        self.head_dim = head_dim
        self.inv_freq = inverse_frequencies(head_dim, theta, scaling)
        self._cos = np.empty((0, head_dim // 2), dtype=np.float32)
        self._sin = np.empty((0, head_dim // 2), dtype=np.float32)
        self._device_tables = {}
        self._retired = []
        if positions:
            self.reserve(positions)

    def reserve(self, positions: int) -> None:
        """Make the table cover positions 0 .. positions-1."""
        have = self._cos.shape[0]
        if positions <= have:
            return
        half = self.head_dim // 2
        cos = np.empty((positions, half), dtype=np.float32)
        sin = np.empty((positions, half), dtype=np.float32)
        cos[:have], sin[:have] = self._cos, self._sin
        cosf, sinf = _libm.cosf, _libm.sinf
        for p in range(have, positions):
            pf = np.float32(p)
            for i in range(half):
                a = float(pf * self.inv_freq[i])  # one 32-bit multiply
                cos[p, i] = cosf(a)
                sin[p, i] = sinf(a)
        self._cos, self._sin = cos, sin
        self._retired.append(self._device_tables)  # captured graphs may still read the old tables
        self._device_tables = {}

    def max_positions(self) -> Optional[int]:
        return self._cos.shape[0]

    def rotary_tables(self, device):
        key = str(device)
        if key not in self._device_tables:
            self._device_tables[key] = (torch.from_numpy(self._cos).to(device),
                                        torch.from_numpy(self._sin).to(device))
        return self._device_tables[key]


class RampScaling:
    """A rescaling of the rotary frequencies for contexts beyond the one a model was trained on: pairs that
    turn fast stay, pairs that turn slowly are divided by ``factor``, a linear ramp over the pair index
    blends between.  With ``index(t) = dims * ln(original / (2 pi t)) / (2 ln base)`` the ramp runs from
    ``lo = max(floor(index(fast)), 0)`` to ``hi = min(ceil(index(slow)), dims - 1)``: ``ramp_i = clamp((i - lo)
    / max(hi - lo, 0.001), 0, 1)`` and the frequency becomes ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``.
    cos and sin are multiplied by ``gain_coefficient * ln(factor) + 1``."""

    def __init__(self, factor: float, original: float, fast: float, slow: float, gain_coefficient: float = 0.1):
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0):
            raise ValueError("a rescaling of rotary frequencies needs positive factor, original, fast and slow")
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        self.gain_coefficient = float(gain_coefficient)

    def key(self):
        return (self.factor, self.original, self.fast, self.slow, self.gain_coefficient)

    def gain(self) -> float:
        return self.gain_coefficient * math.log(self.factor) + 1.0

    def frequencies(self, dims: int, base: float) -> np.ndarray:
        """float64 [dims / 2]."""
        half = dims // 2
        f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)

        def index(turns: float) -> float:
            return dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(index(self.fast)), 0)
        hi = min(math.ceil(index(self.slow)), dims - 1)
        ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / self.factor * ramp + f * (1.0 - ramp)


class HalfRotaryEncoding(RotaryEncoding):
    """Tables for a rotation whose pair i is made of entries i and i + dims / 2 of the turned part (the
    kernels are told the layout; the tables are [positions, dims / 2] either way), with an optional
    :class:`RampScaling`.  Frequencies and angles are formed in 64-bit and rounded once, to the 32-bit
    tables that the kernels read; the tables carry the scaling's gain."""
    layout = "half"

    def __init__(self, dims: int, base: float, scaling: Optional[RampScaling] = None, positions: int = 0):
        if dims % 2 or dims <= 0:
            raise ValueError(f"rotary encoding needs an even number of turned entries, got {dims}")
        if not base > 0:
            raise ValueError("rotary encoding needs a positive base")
        self.head_dim = dims
        self.scaling = scaling
        if scaling is not None:
            self.freq64 = scaling.frequencies(dims, float(base))
            self.gain = scaling.gain()
        else:
            self.freq64 = np.array([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
            self.gain = 1.0
        self.inv_freq = self.freq64.astype(np.float32)
        self._cos = np.empty((0, dims // 2), dtype=np.float32)
        self._sin = np.empty((0, dims // 2), dtype=np.float32)
        self._device_tables = {}
        self._retired = []
        if positions:
            self.reserve(positions)

    def reserve(self, positions: int) -> None:
        have = self._cos.shape[0]
        if positions <= have:
            return
        angles = np.arange(have, positions, dtype=np.float64)[:, None] * self.freq64[None, :]
        self._cos = np.concatenate([self._cos, (np.cos(angles) * self.gain).astype(np.float32)], 0)
        self._sin = np.concatenate([self._sin, (np.sin(angles) * self.gain).astype(np.float32)], 0)
        self._retired.append(self._device_tables)  # captured graphs may still read the old tables
        self._device_tables = {}


register_position_encoding("rotary", RotaryEncoding)
register_position_encoding("rotary_half", HalfRotaryEncoding)
