"""The two ends of a model: token embedding into the residual stream, and the output head.

Embedding rows are multiplied by a scale (``scale_emb``, src/model/embedding.cuh:49-52);
the head multiplies the normed state by a scale (``dim_model_base / hidden_size``,
src/model/linear.cuh:86-104, cpmcu/llm.py:68) and returns fp32 logits.  A tied head uses
the embedding matrix itself; the reference copies it (cpmcu/llm.py:136-137).
"""
from __future__ import annotations

from typing import Dict, Optional, Type

import torch

from .base import Part, Registry, WeightSpec

EMBEDDINGS: Registry[Type[Part]] = Registry("embedding")
HEADS: Registry[Type[Part]] = Registry("output head")


@EMBEDDINGS.register("scaled_embedding")
class ScaledEmbedding(Part):
    recordable_prompt = True

    def __init__(self, ops, vocab_size: int, hidden_size: int, scale: float = 1.0):
        super().__init__(ops)
        self.vocab_size, self.hidden_size, self.scale = int(vocab_size), int(hidden_size), float(scale)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.ops.keep(tensors["weight"].contiguous()) if self.ops is not None else tensors["weight"]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.ops.embed(token_ids, self.weight, self.scale)


@HEADS.register("scaled_lm_head")
class ScaledHead(Part):
    recordable_prompt = True

    def __init__(self, ops, vocab_size: int, hidden_size: int, scale: float = 1.0, tied: bool = False):
        super().__init__(ops)
        self.vocab_size, self.hidden_size, self.scale, self.tied = int(vocab_size), int(hidden_size), float(scale), bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {"weight": WeightSpec((self.vocab_size, self.hidden_size))}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = self.ops.keep(tensors["weight"].contiguous())

    def tie(self, embedding_weight: torch.Tensor) -> None:
        self.weight = embedding_weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        """normed rows [n, hidden] -> fp32 logits [n, vocab]."""
        return self.ops.linear(y, self.weight, alpha=self.scale, out_f32=True, result=True)
