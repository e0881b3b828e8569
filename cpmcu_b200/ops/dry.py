"""The kernel library without a device: every call returns at once and every tensor is a
tensor without storage.

Running the model's own forward pass on it costs microseconds and touches no memory, but it
asks the workspace for exactly the tensors a real step asks for, in the same order and with
the same lifetimes.  That is how the step workspace of the arena is sized: not by a formula
kept beside the model, but by the model's code itself (cpmcu_b200.memory.Workspace counts the
bytes).  The reference sizes its activation area by adding up the layers' ``init_output_ptr``
offsets for ``chunk_length`` tokens (src/model/model.cuh:103-120).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..memory import Arena, Workspace
from ..parts.base import StepContext
from .ops import BF16, F32, Ops, PREFILL_TILE_ROWS


class _NoLibrary:
    """Stands in for the compiled library: every entry point "launches" successfully."""

    @staticmethod
    def cpm_decode_attention_scratch_floats(n_seqs, n_heads, n_kv, d, n_splits):
        return n_seqs * n_kv * ((n_heads // n_kv + 15) // 16) * n_splits * (16 * d + 32)

    @staticmethod
    def cpm_select_blocks_scratch_floats(n_tokens, n_kv, max_entries, n_slices):
        return n_tokens * n_kv * (max_entries * 16 + n_slices * 32)

    @staticmethod
    def cpm_listed_attention_tcgen05_max_pages():
        return 11808

    def __getattr__(self, name):
        return lambda *args: 0


class DryOps(Ops):
    def __init__(self, dtype: torch.dtype, sm_count: int = 148):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.code = F32 if dtype == torch.float32 else BF16
        self.device = torch.device("meta")
        self.lib = _NoLibrary()
        self.element_size = 4 if dtype == torch.float32 else 2
        self.sm_count = sm_count
        self.use_tcgen05 = self.use_tcgen05_attention = self.use_tcgen05_listed = True
        self.tcgen05_pair = False
        arena = Arena(None, None)
        self.workspace = Workspace(arena.carve("persistent", None), [arena.carve("frame0", None), arena.carve("frame1", None)])
        self.weights = None

    # no device, no checks
    @staticmethod
    def _stream():
        return 0

    def _act(self, t, what):
        return t

    @staticmethod
    def _i32(t, what):
        return t

    @staticmethod
    def _f32(t, what):
        return t

    def set_page_limit(self, n_pages):
        pass

    def result(self, *shape, dtype=None):
        return torch.empty(*shape, dtype=dtype or self.dtype, device="meta")


def _meta(n: int) -> torch.Tensor:
    return torch.empty(n, dtype=torch.int32, device="meta")


def dry_context(n_tokens: int, n_seqs: int, max_kv_len: int, cache, decode: bool, captured: bool = False) -> StepContext:
    """A step of ``n_tokens`` tokens shared out evenly over ``n_seqs`` sequences, on tensors without storage."""
    base, extra = divmod(n_tokens, n_seqs)
    q_lens = [base + (1 if i < extra else 0) for i in range(n_seqs)]
    ctx = StepContext(
        n_tokens=n_tokens, n_seqs=n_seqs, is_decode=decode, captured=captured, q_lens=q_lens,
        kv_lens=[] if captured else [max_kv_len] * n_seqs, slots=[] if captured else list(range(n_seqs)),
        max_q_len=max(q_lens), max_kv_len=max_kv_len, token_ids=_meta(n_tokens), positions=_meta(n_tokens),
        token_seq=_meta(n_tokens), cu_q=_meta(n_seqs + 1), kv_len_dev=_meta(n_seqs), slot_dev=_meta(n_seqs), cache=cache)
    n_tiles = sum((n + PREFILL_TILE_ROWS - 1) // PREFILL_TILE_ROWS for n in q_lens)
    ctx.q_tiles = (_meta(n_tiles), _meta(n_tiles), n_tiles)
    ctx.extras["step_begun"] = True
    return ctx


def measure_workspace(spec, dtype: torch.dtype, max_step_tokens: int, max_batch: int, max_seq_tokens: int,
                      sm_count: int = 148) -> Tuple[int, int, List[str]]:
    """(bytes of the persistent part, bytes of one frame, notes) that the steps of a model need at most: prompts of
    ``max_step_tokens`` packed tokens (one long sequence, many short ones, short chunks after a long history) and
    decode steps of ``max_batch`` sequences, each run once on tensors without storage.  A part that cannot run that
    way (it reads values on the host) is left out of the measurement; what it allocates comes from torch's
    allocator anyway, and the note says so."""
    from ..cache import Cache
    from ..models.model import Model

    ops = DryOps(dtype, sm_count)
    model = Model(spec, ops)
    model.load_weights({name: torch.empty(w.shape, device="meta", dtype=torch.int32 if w.role == "table" else dtype)
                        for name, w in model.weight_specs().items()})
    per_seq = max(64, int(max_seq_tokens))
    cache = Cache(model.cache_needs(), max_tokens=per_seq, dtype=dtype, device="meta", n_slots=max(2, max_batch + 1),
                  max_seq_tokens=per_seq, max_step_tokens=max_step_tokens)
    cases = []
    T = int(max_step_tokens)
    for n in sorted({T, max(1, T // 2), min(T, 512), min(T, 256), min(T, 128), min(T, 64)}):
        cases.append((n, 1, per_seq, False, False))
        cases.append((n, min(n, max_batch), per_seq, False, False))
    b = 1
    while b < max_batch:
        b *= 2
    cases.append((b, b, per_seq, True, True))               # a captured decode step of the largest bucket
    cases.append((max_batch, max_batch, per_seq, True, False))
    notes: List[str] = []
    for n_tokens, n_seqs, kv, decode, captured in cases:
        ops.workspace.begin_step()
        try:
            ctx = dry_context(n_tokens, n_seqs, kv, cache, decode, captured)
            rows = ops.empty(n_tokens, dtype=torch.int32)                  # the step's descriptor: ids, positions, ...
            ops.empty(8 * n_tokens + 4 * n_seqs + 64, dtype=torch.int32)
            model.forward(ctx, rows)
        except Exception as e:                                            # a part that needs real values
            note = f"a part could not be measured without a device ({type(e).__name__}: {str(e)[:80]})"
            if note not in notes:
                notes.append(note)
    persistent, frame = ops.workspace.peaks()
    return persistent, frame, notes
