"""Rotary position encodings.

The reference receives a ready ``inv_freq`` table computed in Python by another
package's rope functions and drops the attention factor they return
(cpmcu/llm.py:181-192); its kernel rotates half-split pairs by position * inv_freq
(src/model/rotary.cuh:6-34).  Here the table and the factor are computed from the
configuration's own keys:

    inv_freq[c] = 1 / (factor[c] * theta^(2c/d))
    factor      = long_factor if max_positions > original_max_positions else short_factor
    magnitude   = sqrt(1 + ln(max_positions/original_max_positions) / ln(original_max_positions))
                  if max_positions > original_max_positions else 1

The factor set is chosen once per model, never per call, so cached keys stay valid
however the tokens are cut into steps.  cos and sin are multiplied by the magnitude.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

from .base import POSITIONS, PositionEncoding


@POSITIONS.register("none")
class NoPosition(PositionEncoding):
    """No position information: queries and keys pass unchanged."""

    recordable_prompt = True

    def __init__(self, ops):
        super().__init__(ops)

    def rotary(self):
        return (None, 1.0, 0)


@POSITIONS.register("rope")
class Rotary(PositionEncoding):
    recordable_prompt = True

    def __init__(self, ops, head_dim: int, theta: float, rot_dim: Optional[int] = None):
        super().__init__(ops)
        self.rot_dim = int(rot_dim if rot_dim is not None else head_dim)
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rotary dimension {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.magnitude = 1.0
        self.inv_freq = self._table(theta, [1.0] * (self.rot_dim // 2))

    def _table(self, theta: float, factors: Sequence[float]) -> torch.Tensor:
        # fp32 arithmetic on the host, in the order the formula is written
        exponent = torch.arange(0, self.rot_dim, 2, dtype=torch.int64).to(torch.float32) / self.rot_dim
        f = torch.tensor([float(x) for x in factors], dtype=torch.float32)
        inv_freq = 1.0 / (f * (float(theta) ** exponent))
        return inv_freq.to(torch.float32).to(self.ops.device if self.ops is not None else "cpu")

    def rotary(self) -> Tuple[torch.Tensor, float, int]:
        return (self.inv_freq, self.magnitude, self.rot_dim)


@POSITIONS.register("longrope")
class LongRotary(Rotary):
    def __init__(self, ops, head_dim: int, theta: float, long_factor: Sequence[float],
                 short_factor: Sequence[float], original_max_positions: int, max_positions: int):
        super().__init__(ops, head_dim, theta)
        extended = max_positions > original_max_positions
        factors = long_factor if extended else short_factor
        if len(factors) != self.rot_dim // 2:
            raise ValueError(f"longrope needs {self.rot_dim // 2} factors, got {len(factors)}")
        self.inv_freq = self._table(theta, factors)
        if extended:
            self.magnitude = math.sqrt(1.0 + math.log(max_positions / original_max_positions)
                                       / math.log(original_max_positions))
