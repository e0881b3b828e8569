"""A model put together from a :class:`ModelSpec`: embedding, blocks run in schedule
order, final norm, output head.  Nothing here names an architecture.

The reference's counterpart is the fixed sequence embedding -> layers -> norm ->
lm_head of src/model/model.cuh:145-176, which computes the head on the last row of a
prompt only; here the caller says at which rows logits are wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..parts.base import (NORMS, Block, CacheNeeds, ModelSpec, ResidualStream, StepContext, WeightSpec, build_block,
                          build_part)
from ..parts.embedding import EMBEDDINGS, HEADS


class Model:
    def __init__(self, spec: ModelSpec, ops):
        self.spec = spec
        self.ops = ops
        self.embedding = build_part(EMBEDDINGS, spec.embedding, ops)
        self.blocks: List[Block] = [build_block(layer, ops) for layer in spec.layers]
        self.final_norm = build_part(NORMS, spec.final_norm, ops)
        self.head = build_part(HEADS, spec.head, ops)
        self.schedule = list(spec.schedule)
        for e in self.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {e.layer}; the model has {len(self.blocks)}")
        written = set()
        for e in self.schedule:
            if e.writes_cache:
                if e.lane in written:
                    raise ValueError(f"cache lane {e.lane} is written by two runs of the schedule")
                written.add(e.lane)
            elif e.lane not in written:
                raise ValueError(f"a run reads cache lane {e.lane} before any run has written it")
        self.loaded = False

    # ---- weights ----
    def _named_parts(self):
        yield self.spec.embedding_name, self.embedding
        for layer, block in zip(self.spec.layers, self.blocks):
            yield layer.prefix, block
        yield self.spec.final_norm_name, self.final_norm
        yield self.spec.head_name, self.head

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for name, spec in part.weight_specs().items():
                out[prefix + name] = spec
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._named_parts():
            part.load_weights({n: tensors[prefix + n] for n in part.weight_specs()})
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)
        self.loaded = True

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a decode step has to read: every run of the schedule reads its
        layer's matrices once, the head's matrix once (embedding rows are not counted)."""
        total = sum(self.blocks[e.layer].weight_bytes() for e in self.schedule)
        return total + self.final_norm.weight_bytes() + self.head.weight_bytes()

    def recordable_prompt(self) -> bool:
        """Whether every part can run a prompt chunk without reading the batch on the host (see Part)."""
        parts = [self.embedding, self.final_norm, self.head]
        for b in self.blocks:
            parts += [p for p in (b, b.mixer, b.feed_forward, b.mixer_norm, b.feed_forward_norm) if p is not None]
        return all(bool(getattr(p, "recordable_prompt", False)) for p in parts)

    # ---- cache ----
    def cache_needs(self) -> List[CacheNeeds]:
        needs: List[Optional[CacheNeeds]] = [None] * self.spec.n_lanes()
        for e in self.schedule:
            n = self.blocks[e.layer].mixer.cache_needs()
            if needs[e.lane] is None or e.writes_cache:
                needs[e.lane] = n
        return [n if n is not None else CacheNeeds() for n in needs]

    # ---- forward ----
    def forward(self, ctx: StepContext, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the model; returns fp32 logits [len(want_rows), vocab],
        or None when no logits are wanted (the cache and the state are updated all the same)."""
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        ops = self.ops
        if not ctx.extras.get("step_begun"):
            ops.begin_step()           # the caller did not lay out the step's workspace itself
        stream = ResidualStream(ops, self.embedding.forward(ctx.token_ids))
        for k, e in enumerate(self.schedule):
            ops.begin_layer(k)         # this run's intermediates replace those of the run before the last
            self.blocks[e.layer].forward(ctx, stream, ctx.cache.lane(e.lane), e.writes_cache)
        ops.end_layers()
        if want_rows is None or want_rows.numel() == 0:
            return None
        y = stream.normed(self.final_norm, rows=want_rows)
        return self.head.forward(y)
