"""Rotary position encoding: float32 cos/sin tables indexed by absolute position.

``inv_freq_i = theta^(-2i / R)`` for ``i < R/2`` in float32, ``angle = p * inv_freq``, one
table row per position (``rapid_llm/modules/rotary_embedding.py:30-37,194-202``).  The
rotation itself (half-split pairs ``(i, i + R/2)``) happens inside the fused
q/k-norm + rotation + cache-write kernel, in float32 in both engine precisions.
Identical tables are shared between the layers that ask for them.
"""

from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

_SHARED: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def rope_tables(rotary_dim: int, theta: float, max_positions: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin, float32 ``[max_positions, rotary_dim / 2]``, computed on the host."""
    exponents = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    inv_freq = 1.0 / (torch.tensor(float(theta), dtype=torch.float32) ** exponents)
    angles = torch.outer(torch.arange(max_positions, dtype=torch.float32), inv_freq)
    return torch.cos(angles), torch.sin(angles)


@POSITION_ENCODINGS.register("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, *, head_dim: int, rotary_dim: int, theta: float, max_positions: int, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.max_positions = float(theta), int(max_positions)
        key = (self.rotary_dim, self.theta, self.max_positions, str(self.device))
        if key not in _SHARED:
            cos, sin = rope_tables(self.rotary_dim, self.theta, self.max_positions)
            _SHARED[key] = (cos.to(self.device).contiguous(), sin.to(self.device).contiguous())
        self.cos, self.sin = _SHARED[key]

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


@POSITION_ENCODINGS.register("none")
class NoPositions(PositionEncoding):
    """No rotation: positions do not enter the scores.  The tables have no columns, and as many rows as
    positions are allowed (the rotation kernel checks a position against the rows)."""

    def __init__(self, *, max_positions: int, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.head_dim, self.rotary_dim, self.max_positions = 0, 0, int(max_positions)
        self.cos = torch.empty((self.max_positions, 0), dtype=torch.float32, device=self.device)
        self.sin = self.cos

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


@POSITION_ENCODINGS.register("rotary_frequencies")
class RotaryFrequencies(PositionEncoding):
    """Rotation without tables: the float32 frequencies ``theta^(-2i / R)``, ``i < R / 2``; a kernel forms the angle
    ``position * frequency`` and its sine and cosine itself, so no length bounds the positions."""

    def __init__(self, *, rotary_dim: int, theta: float, max_positions: int, dtype, device) -> None:
        super().__init__(dtype=dtype, device=device)
        if rotary_dim % 2 or rotary_dim < 0:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and not negative")
        self.rotary_dim, self.theta, self.max_positions = int(rotary_dim), float(theta), int(max_positions)
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64) / max(self.rotary_dim, 1)
        self.inv_freq = (float(theta) ** -exponents).to(torch.float32).to(self.device)
        self.magnitude = 1.0       # what cosine and sine are multiplied by

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        raise ValueError("this position encoding has no tables; its kernel computes the angles")


@POSITION_ENCODINGS.register("yarn_frequencies")
class YarnFrequencies(RotaryFrequencies):
    """Frequencies stretched for contexts longer than the ``original`` one: the slow ones divided by ``factor``, the
    fast ones kept, a linear ramp in between.  With ``d(t) = R ln(original / (2 pi t)) / (2 ln theta)`` the index
    at which a frequency turns ``t`` times over the original context, ``lo = max(floor(d(fast)), 0)``,
    ``hi = min(ceil(d(slow)), R - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency is
    ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``; cosine and sine are multiplied by ``0.1 ln(factor) + 1``."""

    def __init__(self, *, rotary_dim: int, theta: float, max_positions: int, factor: float, original: float,
                 fast: float, slow: float, dtype, device) -> None:
        super().__init__(rotary_dim=rotary_dim, theta=theta, max_positions=max_positions, dtype=dtype, device=device)
        import math

        size = self.rotary_dim

        def turns_at(turns: float) -> float:
            return size * math.log(float(original) / (2.0 * math.pi * float(turns))) / (2.0 * math.log(float(theta)))

        lo = max(math.floor(turns_at(fast)), 0)
        hi = min(math.ceil(turns_at(slow)), size - 1)
        index = torch.arange(size // 2, dtype=torch.float64)
        ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        plain = float(theta) ** -(torch.arange(0, size, 2, dtype=torch.float64) / max(size, 1))
        self.inv_freq = (plain / float(factor) * ramp + plain * (1.0 - ramp)).to(torch.float32).to(self.device)
        self.magnitude = 0.1 * math.log(float(factor)) + 1.0
