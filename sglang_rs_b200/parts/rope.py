"""Rotary position encoding.

inv_freq[i] = theta^(-2i / rotary_dim), computed in 64-bit and stored in 32-bit
(reference: crates/sglang-kernel/src/rotary.rs:72-98); angle = float(pos) * inv_freq[i];
pairs are (i, i + rotary_dim/2) in the half-split ("NeoX") style or (2i, 2i + 1)
interleaved (rotary.rs:216-236).  Default scaling has magnitude 1 (rotary.rs:100-103).
The table is a constant of the model; the rotation itself runs inside the fused q/k
kernel.

:class:`WavelengthScaling` stretches the long wavelengths for contexts beyond the one a model was trained on:
with d(t) = dims * ln(original / (2 pi t)) / (2 ln theta) (the pair whose wavelength makes t turns over the
original context), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and ramp_i = clamp((i - lo) /
max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i * (1 - ramp_i); cosines and sines are
multiplied by 0.1 ln(factor) + 1 (``magnitude``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .base import PositionEncoding


@dataclass(frozen=True)
class FusedRotary:
    """What the fused q/k kernel needs to rotate: either a table ``inv_freq`` (angle = position *
    inv_freq[i]) or ``angles(positions) -> float32 [rows, rotary_dim / 2]`` for encodings whose angles
    are not a product of position and frequency."""
    inv_freq: Optional[torch.Tensor]
    rotary_dim: int
    interleaved: bool
    angles: Optional[Callable[[torch.Tensor], torch.Tensor]] = None
    #: factor on every cosine and sine
    magnitude: float = 1.0


@dataclass(frozen=True)
class WavelengthScaling:
    """Stretching of the long wavelengths of a rotary table (see the module's text)."""
    factor: float
    original: float          # positions of the original context
    fast: float              # pairs that make more turns than this over the original context keep their frequency
    slow: float              # pairs that make fewer turns than this are slowed by ``factor``

    def __post_init__(self):
        if not (self.factor > 0 and self.original > 0 and self.fast > 0 and self.slow > 0):
            raise ValueError("rotary scaling needs a positive factor, context and turn counts")

    @property
    def magnitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0

    def apply(self, frequencies: torch.Tensor, rotary_dim: int, theta: float) -> torch.Tensor:
        """``frequencies`` float64 [rotary_dim / 2] -> the stretched ones."""
        def pair_of(turns: float) -> float:
            return rotary_dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
        lo = max(math.floor(pair_of(self.fast)), 0)
        hi = min(math.ceil(pair_of(self.slow)), rotary_dim - 1)
        index = torch.arange(frequencies.numel(), dtype=torch.float64)
        ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return frequencies / self.factor * ramp + frequencies * (1.0 - ramp)


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    fused = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, interleaved: bool = False,
                 scaling: Optional[WavelengthScaling] = None):
        self.head_dim = int(head_dim)
        self.scaling = scaling
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        self.theta = float(theta)
        self.interleaved = bool(interleaved)
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rotary_dim} must be even, positive and at most {self.head_dim}")
        if not self.theta > 0:
            raise ValueError("RoPE theta must be finite and positive")
        if scaling is not None and not self.theta > 1:
            raise ValueError("rotary scaling needs a base above 1")
        self._table: Optional[FusedRotary] = None

    def inverse_frequencies(self) -> torch.Tensor:
        pair = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        frequencies = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * pair / self.rotary_dim)
        if self.scaling is not None:
            frequencies = self.scaling.apply(frequencies, self.rotary_dim, self.theta)
        return frequencies.to(torch.float32)

    def load(self, tensors, device, dtype) -> None:
        # an encoding that several layers share is loaded once: they then share one table on the device
        if self._table is None or self._table.inv_freq.device != torch.device(device):
            self._table = FusedRotary(self.inverse_frequencies().to(device), self.rotary_dim, self.interleaved,
                                      magnitude=self.scaling.magnitude if self.scaling is not None else 1.0)

    def fused_rotary(self) -> FusedRotary:
        return self._table


class NoPositionEncoding(PositionEncoding):
    """Leaves q and k as they are."""
    graph_safe = True

    fused = True

    def fused_rotary(self):
        return None
