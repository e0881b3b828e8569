"""Gated feed-forward: down( act(gate(y)) * up(y) ) (src/model/ffn.cuh:18-89).

gate and up are kept as one [2*inter, hidden] matrix so that one product gives both
(src/model/ffn.cuh:47-48 keeps them as [gate | up]; here their rows are interleaved in
blocks of 8 when the size allows); the activation is SiLU in fp32
(src/model/activation.cuh:6-18)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, FeedForward, WeightSpec


@FEED_FORWARDS.register("gated_ffn")
class GatedFeedForward(FeedForward):
    recordable_prompt = True

    def __init__(self, ops, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        super().__init__(ops)
        if activation != "silu":
            raise ValueError(f"gated_ffn: activation '{activation}' is not built; known: ['silu']")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.interleave = 0
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
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        i, h = self.intermediate_size, self.hidden_size
        if i % 8 == 0:
            # blocks of 8 gate rows followed by the 8 up rows of the same features: gate and up of a
            # feature then fall into one tile of the product, which can apply the activation itself
            self.interleave = 8
            self.w_gate_up = torch.stack([gate.view(i // 8, 8, h), up.view(i // 8, 8, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            self.interleave = 0
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_gate_up = self.ops.keep(self.w_gate_up)
        self.w_down = self.ops.keep(tensors["down_proj.weight"].contiguous())

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_gate_up.element_size()

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        h = self.ops.gated_linear(y, self.w_gate_up, self.interleave)
        return self.ops.linear(h, self.w_down)
