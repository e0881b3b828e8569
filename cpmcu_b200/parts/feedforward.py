"""Gated feed-forward: down( act(gate(y)) * up(y) ) (src/model/ffn.cuh:18-89).

gate and up are kept as one [2*inter, hidden] matrix so that one product gives a row
[gate | up] (src/model/ffn.cuh:47-48); the activation is SiLU in fp32
(src/model/activation.cuh:6-18)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, FeedForward, WeightSpec


@FEED_FORWARDS.register("gated_ffn")
class GatedFeedForward(FeedForward):
    def __init__(self, ops, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        super().__init__(ops)
        if activation != "silu":
            raise ValueError(f"gated_ffn: activation '{activation}' is not built; known: ['silu']")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        i, h = self.intermediate_size, self.hidden_size
        return {
            "gate_proj.weight": WeightSpec((i, h)),
            "up_proj.weight": WeightSpec((i, h)),
            "down_proj.weight": WeightSpec((h, i)),
        }

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_gate_up.element_size()

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        gu = self.ops.linear(y, self.w_gate_up)
        h = self.ops.silu_mul(gu)
        return self.ops.linear(h, self.w_down)
