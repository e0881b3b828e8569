"""The step function: one batch of sequences, the tokens each brings, logits where wanted.

A step runs only the tokens it is given, as one packed batch, against the cache
that earlier steps left: prompts of unequal lengths in one step (cut into chunks of
at most ``chunk_tokens`` packed tokens when long), then one token per sequence.
The reference has two entry points for one sequence, ``prefill`` (logits of the
last row) and ``decode`` (src/model/model.cuh:156-176), and a Python loop that chunks
a prompt (cpmcu/llm.py:212-218).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache import Cache
from ..models.model import Model
from ..ops.ops import PREFILL_TILE_ROWS
from ..parts.base import StepContext


@dataclass
class SequenceStep:
    """What one sequence brings to a step: its slot, its next tokens, and the places
    among these tokens whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class Chunk:
    """A contiguous piece [begin, end) of the step's packed token axis."""

    begin: int
    end: int
    pieces: List[Tuple[int, int, int]] = field(default_factory=list)   # (sequence index, first token, count)


def plan_chunks(lengths: Sequence[int], chunk_tokens: int) -> List[Chunk]:
    """Cuts the packed token axis of sequences with ``lengths`` into chunks of at most
    ``chunk_tokens`` tokens.  A sequence may continue in the next chunk."""
    if chunk_tokens <= 0:
        raise ValueError("chunk_tokens must be positive")
    chunks: List[Chunk] = []
    cur = Chunk(0, 0)
    pos = 0
    for i, n in enumerate(lengths):
        done = 0
        while done < n:
            room = chunk_tokens - (cur.end - cur.begin)
            if room == 0:
                chunks.append(cur)
                cur = Chunk(pos, pos)
                room = chunk_tokens
            take = min(room, n - done)
            cur.pieces.append((i, done, take))
            cur.end += take
            pos += take
            done += take
    if cur.end > cur.begin:
        chunks.append(cur)
    return chunks


class Stepper:
    """Drives a model over a cache, step by step."""

    def __init__(self, model: Model, cache: Cache, chunk_tokens: int = 2048):
        self.model = model
        self.cache = cache
        self.ops = model.ops
        self.chunk_tokens = int(chunk_tokens)
        self.vocab_size = model.spec.vocab_size
        self.taps: Optional[dict] = None      # when set, parts may leave intermediate results in it (ctx.extras["taps"])

    # ---- sequences ----
    def open(self, n: int) -> List[int]:
        return self.cache.open_sequences(n)

    def close(self, slot: int) -> None:
        self.cache.close_sequence(slot)

    # ---- one step ----
    def step(self, batch: Sequence[SequenceStep]) -> Optional[torch.Tensor]:
        """Returns fp32 logits [total wanted, vocab] in the order of the batch and of each
        ``want``, or None if nothing is wanted."""
        if not batch:
            return None
        seen = set()
        for s in batch:
            if s.slot in seen:
                raise ValueError(f"slot {s.slot} appears twice in one step")
            seen.add(s.slot)
            if len(s.tokens) == 0:
                raise ValueError(f"slot {s.slot} brings no tokens")
            for t in s.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise ValueError(f"token id {t} is outside the vocabulary [0, {self.vocab_size})")
            for w in s.want:
                if not 0 <= int(w) < len(s.tokens):
                    raise ValueError(f"wanted place {w} is outside the {len(s.tokens)} tokens of slot {s.slot}")
        lengths = [len(s.tokens) for s in batch]
        history = [self.cache.length(s.slot) for s in batch]
        chunks = plan_chunks(lengths, self.chunk_tokens)
        # One chunk: room for the whole step is taken before anything runs.  Several chunks: the room is checked
        # before anything runs and taken chunk by chunk, so that layers with a window can give pages back on the way.
        if len(chunks) == 1:
            for s, h, n in zip(batch, history, lengths):
                self.cache.reserve(s.slot, h + n)
            self.cache.sync()
        else:
            self.cache.check_room([(s.slot, h + n) for s, h, n in zip(batch, history, lengths)], self.chunk_tokens)

        # wanted rows in packed coordinates, in request order
        offsets = [0]
        for n in lengths:
            offsets.append(offsets[-1] + n)
        wanted: List[int] = [offsets[i] + int(w) for i, s in enumerate(batch) for w in s.want]
        logits: Optional[torch.Tensor] = None
        if wanted:
            logits = torch.empty(len(wanted), self.vocab_size, dtype=torch.float32, device=self.ops.device)

        for chunk in chunks:
            rows_here = [(k, p - chunk.begin) for k, p in enumerate(wanted) if chunk.begin <= p < chunk.end]
            if len(chunks) > 1:
                for i, first, count in chunk.pieces:
                    self.cache.reserve(batch[i].slot, history[i] + first + count)
                self.cache.sync()
            out = self._run_chunk(batch, history, chunk, [r for _, r in rows_here])
            if len(chunks) > 1:
                for i, first, count in chunk.pieces:
                    self.cache.set_length(batch[i].slot, history[i] + first + count)
            if rows_here:
                if len(chunks) == 1 and len(rows_here) == len(wanted):
                    logits = out
                else:
                    idx = torch.tensor([k for k, _ in rows_here], dtype=torch.int64, device=self.ops.device)
                    logits.index_copy_(0, idx, out)
        for s, h, n in zip(batch, history, lengths):
            self.cache.set_length(s.slot, h + n)
        return logits

    def _run_chunk(self, batch, history, chunk: Chunk, want_rows: List[int]) -> Optional[torch.Tensor]:
        ids: List[int] = []
        positions: List[int] = []
        token_seq: List[int] = []
        cu_q = [0]
        kv_lens: List[int] = []
        q_lens: List[int] = []
        slots: List[int] = []
        for j, (i, first, count) in enumerate(chunk.pieces):
            s = batch[i]
            ids.extend(int(t) for t in s.tokens[first:first + count])
            start = history[i] + first
            positions.extend(range(start, start + count))
            token_seq.extend([j] * count)
            cu_q.append(cu_q[-1] + count)
            kv_lens.append(start + count)
            q_lens.append(count)
            slots.append(s.slot)
        n_tok, n_seq = len(ids), len(slots)
        ws = self.ops.workspace
        if ws is not None:
            ws.require(n_tok, n_seq)          # a step the workspace was not sized for is refused before anything runs
        self.ops.begin_step()
        # query tiles of the prefill attention kernel: (sequence, first token of the tile)
        tile_seq = [j for j, n in enumerate(q_lens) for _ in range(0, n, PREFILL_TILE_ROWS)]
        tile_row = [r for n in q_lens for r in range(0, n, PREFILL_TILE_ROWS)]
        packed = torch.tensor(ids + positions + token_seq + cu_q + kv_lens + slots + want_rows + tile_seq + tile_row,
                              dtype=torch.int32)
        dev = self.ops.empty(packed.numel(), dtype=torch.int32)
        dev.copy_(packed)                     # pageable staging: the copy is over when this returns
        o = 0

        def cut(n: int) -> torch.Tensor:
            nonlocal o
            t = dev[o:o + n]
            o += n
            return t

        ctx = StepContext(
            n_tokens=n_tok, n_seqs=n_seq, is_decode=all(q == 1 for q in q_lens), captured=False,
            q_lens=q_lens, kv_lens=kv_lens, slots=slots, max_q_len=max(q_lens), max_kv_len=max(kv_lens),
            token_ids=cut(n_tok), positions=cut(n_tok), token_seq=cut(n_tok), cu_q=cut(n_seq + 1),
            kv_len_dev=cut(n_seq), slot_dev=cut(n_seq), cache=self.cache,
        )
        rows = cut(len(want_rows)) if want_rows else None
        ctx.extras["q_tiles"] = (cut(len(tile_seq)), cut(len(tile_row)), len(tile_seq))
        ctx.extras["step_begun"] = True
        if self.taps is not None:
            ctx.extras["taps"] = self.taps
        return self.model.forward(ctx, rows)
