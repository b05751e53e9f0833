"""Rotary position encoding with rotate-half pairing (element i with i + rotary_dim/2).

The angles follow crates/coheryn-engine/src/cpu.rs:58-73 exactly: in float32,
``step = theta ** (-2 / head_dim)``, ``angle_0 = position`` and
``angle_{i+1} = angle_i * step`` (an iterated product, not ``position * theta**(-2i/d)``;
the two differ by about 1e-4 at a few hundred positions).  cos and sin of every
(position, pair) are tabulated once when the model is built; the kernels only look
them up.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Position, Runtime, register_position


class RotateHalfRope(Position):
    def __init__(self, runtime: Runtime, head_dim: int, rotary_dim: int, theta: float,
                 max_positions: int):
        super().__init__(runtime)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.max_positions = float(theta), int(max_positions)
        self._table = None

    def angle_table(self) -> np.ndarray:
        """float32 [max_positions, rotary_dim/2] of angles, by the iterated product."""
        half = self.rotary_dim // 2
        step = np.float32(np.power(np.float32(self.theta), np.float32(-2.0) / np.float32(self.rotary_dim)))
        angles = np.empty((self.max_positions, half), dtype=np.float32)
        a = np.arange(self.max_positions, dtype=np.float32)
        for i in range(half):
            angles[:, i] = a
            a = (a * step).astype(np.float32)
        return angles

    def cos_sin(self) -> torch.Tensor:
        """float32 [max_positions, rotary_dim/2, 2] = (cos, sin) on the device."""
        if self._table is None:
            ang = self.angle_table()
            t = np.stack([np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)], axis=-1)
            self._table = torch.from_numpy(np.ascontiguousarray(t)).to(self.runtime.device)
        return self._table


class ComputedRope(Position):
    """Rotate-half rotary encoding whose angles the kernels compute from the position (no table, so no bound on
    positions): pair i of the first ``rotary_dim`` channels turns by position * f_i, f_i = theta^(-2i / rotary_dim).

    ``scaling`` (optional) is the YaRN interpolation by parts: with d(t) = rotary_dim * ln(original / (2 pi t)) /
    (2 ln theta), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency becomes f_i / factor * ramp_i + f_i (1 - ramp_i)
    and cos and sin are multiplied by 0.1 ln(factor) + 1.

    The frequencies are made in float64 and handed to the device as a float32 pair (high, low) each; the kernel
    forms position * (high + low) without losing the low part, so the angle is good to float32's last bit at any
    position."""

    def __init__(self, runtime: Runtime, rotary_dim: int, theta: float, scaling=None):
        super().__init__(runtime)
        if rotary_dim % 2 or rotary_dim < 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and positive")
        if not theta > 1:
            raise ValueError("the base of the frequencies must exceed 1")
        self.rotary_dim, self.theta = int(rotary_dim), float(theta)
        self.scaling = dict(scaling) if scaling else None
        if self.scaling is not None:
            for key in ("factor", "original", "fast", "slow"):
                if not float(self.scaling.get(key, 0)) > 0:
                    raise ValueError(f"rotary scaling needs a positive {key!r}")
        self._freq = None

    def frequencies(self) -> np.ndarray:
        """float64 [rotary_dim / 2]."""
        import math
        dims, half = self.rotary_dim, self.rotary_dim // 2
        i = np.arange(half, dtype=np.float64)
        f = np.power(np.float64(self.theta), -2.0 * i / dims)
        if self.scaling is not None:
            s = self.scaling
            where = lambda t: dims * math.log(float(s["original"]) / (2.0 * math.pi * float(t))) / (2.0 * math.log(self.theta))
            lo = max(math.floor(where(s["fast"])), 0)
            hi = min(math.ceil(where(s["slow"])), dims - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / float(s["factor"]) * ramp + f * (1.0 - ramp)
        return f

    @property
    def amplitude(self) -> float:
        """What cos and sin are multiplied by."""
        import math
        return 0.1 * math.log(float(self.scaling["factor"])) + 1.0 if self.scaling is not None else 1.0

    def frequency_pairs(self) -> torch.Tensor:
        """float32 [rotary_dim / 2, 2] on the device: each frequency as high + low."""
        if self._freq is None:
            f = self.frequencies()
            high = f.astype(np.float32)
            low = (f - high.astype(np.float64)).astype(np.float32)
            self._freq = torch.from_numpy(np.ascontiguousarray(np.stack([high, low], axis=-1))).to(self.runtime.device)
        return self._freq


register_position("rope_rotate_half", RotateHalfRope)
register_position("rope_computed", ComputedRope)
