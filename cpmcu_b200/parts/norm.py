"""RMS norm (src/model/norm.cuh:7-51): y = x * rsqrt(mean(x^2) + eps) * weight, the weight
used as it is stored (not 1 + weight)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, Norm, WeightSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    recordable_prompt = True

    def __init__(self, ops, hidden_size: int, eps: float):
        super().__init__(ops)
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.hidden_size,), "vector")}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.ops.keep(tensors["weight"].contiguous())

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.add_rmsnorm(x, None, 0.0, self.weight, self.eps, rows)

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, scale: float,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.add_rmsnorm(x, delta, scale, self.weight, self.eps, rows)
