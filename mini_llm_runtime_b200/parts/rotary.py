"""Rotary position encoding as a table of cosines and sines.

`freq_j = theta^(-2j/D)`, `angle = float(position) * freq_j`, all in float32, as
src/minillm/runtime.cpp:231-241 computes them for each step and
src/minillm/cuda/storage.cpp:261-287 tabulates them once ([positions, D], cosines
in the first half of a row, sines in the second).  The table is made on the host
with float32 `pow`, multiply, `cos` and `sin`, then uploaded; the mixer's kernel
rotates `(x[j], x[j + D/2])` pairs with it.
Parameters: theta, rotary_dim, max_positions.  No weights.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..config.registry import register_part
from .base import PositionEncoding


def rotation_table(theta: float, rotary_dim: int, max_positions: int) -> torch.Tensor:
    half = rotary_dim // 2
    j = np.arange(half, dtype=np.float32)
    exponent = (np.float32(-2.0) * j / np.float32(rotary_dim)).astype(np.float32)
    freq = np.power(np.float32(theta), exponent).astype(np.float32)
    pos = np.arange(max_positions, dtype=np.float32)[:, None]
    angle = (pos * freq[None, :]).astype(np.float32)
    table = np.concatenate([np.cos(angle), np.sin(angle)], axis=1).astype(np.float32)
    return torch.from_numpy(table)


class Rope(PositionEncoding):
    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        self._table: Optional[torch.Tensor] = None

    def bind(self, tensors, rt) -> None:
        self._table = rotation_table(self.theta, self.rotary_dim, self.max_positions).to(rt.device)

    def rotation_table(self) -> Optional[torch.Tensor]:
        return self._table


register_part("position", "rope", Rope)


def scaled_frequencies(freq: np.ndarray, factor: float, low: float, high: float, original: float) -> np.ndarray:
    """Frequencies whose long wavelengths are slowed down, as a model does that was trained on `original` positions and
    is to read `factor` times as many: with the wavelength l = 2 pi / f, a frequency stays where l < original / high,
    becomes f / factor where l > original / low, and in between is the blend (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low).  float64 in, float64 out."""
    freq = np.asarray(freq, dtype=np.float64)
    length = 2.0 * np.pi / freq
    s = (original / length - low) / (high - low)
    blend = (1.0 - s) * freq / factor + s * freq
    return np.where(length < original / high, freq, np.where(length > original / low, freq / factor, blend))


class RotaryFrequencies(PositionEncoding):
    """Rotation given as its frequencies only: `freq_i = base^(-2i/dims) / factor`, i < dims/2.  The kernels
    that use it compute `position * freq_i` and its cosine and sine in float32 themselves, so no table
    exists and no largest position: `factor` > 1 is linear position scaling.  Only the first `dims`
    values of a head are rotated; a mixer's heads may be wider.  Value i turns with value i + dims/2, or, with
    `interleaved`, value 2i with value 2i + 1: (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freq_i
    (a mixer's kernels must know that layout; those that do not refuse it).
    With `scaling` = {factor, low, high, original} only long wavelengths are slowed down (`scaled_frequencies`).
    Parameters: base, dims, factor (default 1), interleaved (default False), scaling (default None).  No weights."""

    def __init__(self, spec):
        super().__init__(spec)
        self.base = float(spec.params["base"])
        self.dims = int(spec.params["dims"])
        self.factor = float(spec.params.get("factor", 1.0))
        self.interleaved = bool(spec.params.get("interleaved", False))
        if self.dims < 0 or self.dims % 2 or self.base <= 0 or self.factor <= 0:
            raise ValueError(f"a rotation of {self.dims} values with base {self.base} and factor {self.factor} is not defined")
        scaling = spec.params.get("scaling")
        self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")} if scaling else None
        if self.scaling is not None and not (self.scaling["high"] > self.scaling["low"] and self.scaling["factor"] > 0
                                             and self.scaling["original"] > 0):
            raise ValueError(f"a frequency scaling {self.scaling} is not defined")
        self._freq: Optional[torch.Tensor] = None

    def bind(self, tensors, rt) -> None:
        i = np.arange(self.dims // 2, dtype=np.float64)
        freq = np.power(self.base, -2.0 * i / max(self.dims, 1)) / self.factor
        if self.scaling is not None:
            freq = scaled_frequencies(freq, **self.scaling)
        self._freq = torch.from_numpy(freq.astype(np.float32)).to(rt.device)

    def frequencies(self) -> torch.Tensor:
        return self._freq


register_part("position", "rotary_frequencies", RotaryFrequencies)
