"""Lays a model's storage out in one arena: weights, the step workspace, per-sequence state
and key-value pages (cpmcu_b200.memory).

The reference does this in ``init_storage`` (src/model/model.cuh:103-120): weights first,
the activation area for ``chunk_length`` tokens next, the cache takes the rest.  Here the
workspace is measured by running the model once on tensors without storage
(cpmcu_b200.ops.dry), and the cache's bytes by building its tables the same way.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..cache import Cache, PAGE_TOKENS
from ..memory import ALIGN, Arena, PoolExhausted, Workspace, plan_storage, round_up
from ..models.model import Model
from ..ops.dry import measure_workspace
from .decode import bucket_size


@dataclass
class Storage:
    arena: Arena
    cache: Cache
    workspace: Workspace
    tokens: int
    notes: List[str] = field(default_factory=list)

    def report(self) -> str:
        rows = [f"{name}: {size / 2**20:,.1f} MiB" for name, (size, _) in self.arena.report().items()]
        return f"arena {self.arena.total / 2**20:,.1f} MiB = " + ", ".join(rows)


def weight_bytes(model: Model) -> int:
    """Bytes the model's weights take in the arena (vectors counted as 32-bit, the most they can be)."""
    es = model.ops.element_size
    total = 0
    for spec in model.weight_specs().values():
        n = 1
        for s in spec.shape:
            n *= s
        total += round_up(n * (es if spec.role == "matrix" else 4))
    return total + 64 * ALIGN


def make_storage(model: Model, chunk_tokens: int, max_batch: int, max_tokens: Optional[int] = None,
                 memory_limit: Optional[float] = None, max_seq_tokens: Optional[int] = None,
                 n_slots: Optional[int] = None, reserve_bytes: int = 512 << 20) -> Storage:
    """One arena for ``model``: attaches the weight region and the workspace to the model's ``ops`` and returns the
    cache made inside it.  ``max_tokens``: the tokens the cache holds; without it the cache takes what
    ``memory_limit`` (a fraction of the device's memory) leaves after weights, workspace and ``reserve_bytes`` (for
    what torch allocates itself: results handed to callers, library workspaces).  Weights that are already loaded
    stay where they are; otherwise they go into the arena when they are loaded.  Raises PoolExhausted."""
    ops = model.ops
    spec = model.spec
    dtype, device = ops.dtype, ops.device
    needs = model.cache_needs()
    bucket = bucket_size(max_batch)
    per_seq_cap = max_seq_tokens or max(spec.max_positions, 4096) * 8

    def slots_for(tokens: int) -> int:
        return n_slots or min(max(2, tokens // PAGE_TOKENS), max_batch * 2 + 2)

    def counted_cache(tokens: int):
        counting = Arena(None, None)
        st, pg = counting.carve("state", None), counting.carve("cache", None)
        Cache(needs, max_tokens=tokens, dtype=dtype, device="meta", n_slots=slots_for(tokens),
              max_seq_tokens=min(tokens, per_seq_cap), max_step_tokens=chunk_tokens, state_region=st, page_region=pg)
        return round_up(st.peak) + 16 * ALIGN, round_up(pg.peak) + 16 * ALIGN

    persistent, frame, notes = measure_workspace(spec, dtype, chunk_tokens, max_batch, per_seq_cap, ops.sm_count)
    persistent = round_up(int(persistent * 1.05) + (1 << 20))
    frame = round_up(int(frame * 1.05) + (1 << 20))
    w_bytes = 0 if model.loaded else weight_bytes(model)
    budget = None
    if max_tokens is None:
        if memory_limit is None:
            raise ValueError("make_storage needs max_tokens or memory_limit")
        free, total = torch.cuda.mem_get_info(device)
        budget = min(free, int(total * float(memory_limit))) - int(reserve_bytes)
        if budget <= 0:
            raise PoolExhausted("arena", reserve_bytes, min(free, int(total * float(memory_limit))), 0,
                                f"memory_limit {memory_limit} of {total >> 20} MiB ({free >> 20} MiB free) leaves nothing")
    tokens, total_bytes = plan_storage(budget, w_bytes, persistent + 2 * frame, lambda t: sum(counted_cache(t)), max_tokens)
    st_bytes, pg_bytes = counted_cache(tokens)
    checked = os.environ.get("CPMCU_CHECK_BOUNDS", "0") not in ("", "0")       # guard words behind every region
    total_bytes = w_bytes + persistent + 2 * frame + st_bytes + pg_bytes + 16 * ALIGN      # what the regions add up to
    arena = Arena(total_bytes, device, guards=checked)
    if w_bytes:
        ops.weights = arena.carve("weights", w_bytes)
    workspace = Workspace(arena.carve("workspace", persistent), [arena.carve("frame0", frame), arena.carve("frame1", frame)],
                          sized_tokens=max(chunk_tokens, bucket), sized_seqs=max(bucket, 1))
    cache = Cache(needs, max_tokens=tokens, dtype=dtype, device=device, n_slots=slots_for(tokens),
                  max_seq_tokens=min(tokens, per_seq_cap), max_step_tokens=chunk_tokens,
                  state_region=arena.carve("state", st_bytes), page_region=arena.carve("cache", pg_bytes))
    ops.workspace = workspace
    return Storage(arena, cache, workspace, tokens, notes)
