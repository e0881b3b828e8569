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

import numpy as np
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


MAX_GRAPH_PIECES = 16        # most sequences whose pieces a recorded chunk may hold


class _PromptGraph:
    """A recorded prompt chunk: its input buffer [ids | positions | keys after the chunk, slot | wanted rows], the
    buffers that never change (token -> sequence, offsets, query tiles), the graph and its logits."""

    def __init__(self, inputs: torch.Tensor, fixed: torch.Tensor):
        self.inputs, self.fixed = inputs, fixed
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None


class Stepper:
    """Drives a model over a cache, step by step."""

    def __init__(self, model: Model, cache: Cache, chunk_tokens: int = 2048, graph_prompts: bool = False):
        """``graph_prompts``: a full chunk of prompt tokens (``chunk_tokens`` tokens: all chunks of a long prompt but the
        last, and the full chunks of a batch of prompts, which hold pieces of up to MAX_GRAPH_PIECES sequences) is
        recorded into a CUDA graph the first time its kind runs and replayed from then on, whatever the sequences and
        their histories, because every kernel reads lengths, positions, offsets and pages from device memory.  It takes
        the host out of the prompt (about ten launches a layer otherwise) and needs a model whose parts are all
        ``recordable_prompt``."""
        self.model = model
        self.cache = cache
        self.ops = model.ops
        self.chunk_tokens = int(chunk_tokens)
        self.vocab_size = model.spec.vocab_size
        self.taps: Optional[dict] = None      # when set, parts may leave intermediate results in it (ctx.extras["taps"])
        self.graph_prompts = bool(graph_prompts) and model.recordable_prompt()
        # recorded chunks by (tokens, wanted rows, bound on the sequences' lengths, pieces of several sequences?)
        self.prompt_graphs: Dict[Tuple[int, int, int, bool], "_PromptGraph"] = {}

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
        arrays: List[np.ndarray] = []                       # every sequence's tokens, checked once, as int32
        for s in batch:
            if s.slot in seen:
                raise ValueError(f"slot {s.slot} appears twice in one step")
            seen.add(s.slot)
            if len(s.tokens) == 0:
                raise ValueError(f"slot {s.slot} brings no tokens")
            arr = np.asarray(s.tokens, dtype=np.int64)
            if arr.ndim != 1:
                raise ValueError(f"slot {s.slot}: tokens must be a flat sequence of ids")
            if int(arr.min()) < 0 or int(arr.max()) >= self.vocab_size:
                bad = int(arr[(arr < 0) | (arr >= self.vocab_size)][0])
                raise ValueError(f"token id {bad} is outside the vocabulary [0, {self.vocab_size})")
            arrays.append(arr.astype(np.int32))
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
            out = self._run_chunk(batch, arrays, history, chunk, [r for _, r in rows_here])
            if len(chunks) > 1:
                for i, first, count in chunk.pieces:
                    self.cache.set_length(batch[i].slot, history[i] + first + count)
            if rows_here:
                if len(chunks) == 1 and len(rows_here) == len(wanted):
                    logits = out
                else:
                    ks = [k for k, _ in rows_here]
                    if ks == list(range(ks[0], ks[0] + len(ks))):          # the usual case: one plain copy
                        logits[ks[0]:ks[0] + len(ks)].copy_(out)
                    else:
                        logits.index_copy_(0, torch.tensor(ks, dtype=torch.int64, device=self.ops.device), out)
        for s, h, n in zip(batch, history, lengths):
            self.cache.set_length(s.slot, h + n)
        return logits

    def _graph_chunk(self, tokens: np.ndarray, slot: int, start: int, want_rows: List[int]) -> Optional[torch.Tensor]:
        """A full chunk of one sequence through its recorded graph; None if there is none yet (the chunk then runs
        the ordinary way, and is recorded afterwards for the chunks to come)."""
        n = int(tokens.shape[0])
        g = self.prompt_graphs[(n, len(want_rows), self._length_bound(start + n), False)]
        host = np.concatenate([tokens, np.arange(start, start + n, dtype=np.int32),
                               np.asarray([start + n, slot] + list(want_rows), dtype=np.int32)])
        g.inputs.copy_(torch.from_numpy(host))
        g.graph.replay()
        return None if g.logits is None else g.logits.clone()

    def _length_bound(self, kv_len: int) -> int:
        """The bound on the sequence's length that a recorded chunk is made for: the next power of two (at least
        1,024), at most the cache's capacity per sequence.  Parts decide on the host from this bound (which kernel,
        how many shares, dense or sparse attention), so a recording serves every chunk below its bound."""
        bound = 1024
        while bound < kv_len:
            bound *= 2
        return min(bound, self.cache.max_pages_per_seq * 64)

    def _record_chunk(self, n: int, n_want: int, bound: int) -> None:
        """Records the graph of a full chunk of ``n`` tokens with ``n_want`` wanted rows for sequences of up to
        ``bound`` tokens.  Nothing runs: the recording's own launches are never executed."""
        ops, dev = self.ops, self.ops.device
        inputs = torch.zeros(2 * n + 2 + n_want, dtype=torch.int32, device=dev)
        n_tiles = (n + PREFILL_TILE_ROWS - 1) // PREFILL_TILE_ROWS
        fixed = torch.cat([torch.zeros(n, dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32),
                           torch.zeros(n_tiles, dtype=torch.int32),
                           torch.arange(0, n, PREFILL_TILE_ROWS, dtype=torch.int32)]).to(dev)
        g = _PromptGraph(inputs, fixed)
        def body():
            ws = ops.workspace
            if ws is not None:
                ws.require(n, 1)
            ops.begin_step()
            ctx = StepContext(
                n_tokens=n, n_seqs=1, is_decode=(n == 1), captured=True, q_lens=[n], kv_lens=[], slots=[], max_q_len=n,
                max_kv_len=bound, token_ids=inputs[:n], positions=inputs[n:2 * n], token_seq=fixed[:n],
                cu_q=fixed[n:n + 2], kv_len_dev=inputs[2 * n:2 * n + 1], slot_dev=inputs[2 * n + 1:2 * n + 2], cache=self.cache)
            ctx.q_tiles = (fixed[n + 2:n + 2 + n_tiles], fixed[n + 2 + n_tiles:], n_tiles)
            ctx.extras["step_begun"] = True
            return self.model.forward(ctx, inputs[2 * n + 2:] if n_want else None)

        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            g.logits = body()
        g.graph = graph
        self.prompt_graphs[(n, n_want, bound, False)] = g

    def _run_chunk(self, batch, arrays, history, chunk: Chunk, want_rows: List[int]) -> Optional[torch.Tensor]:
        record = None
        if self.graph_prompts and self.taps is None and chunk.end - chunk.begin == self.chunk_tokens and self.chunk_tokens > 1 \
                and len(chunk.pieces) <= MAX_GRAPH_PIECES:
            packed = len(chunk.pieces) > 1
            ws = self.ops.workspace
            if packed and ws is not None and ws.sized_seqs and ws.sized_seqs < MAX_GRAPH_PIECES + 1:
                return self._run_chunk_eager(batch, arrays, history, chunk, want_rows)      # a workspace made for fewer sequences
            bound = self._length_bound(max(history[i] + first + count for i, first, count in chunk.pieces))
            key = (self.chunk_tokens, len(want_rows), bound, packed)
            if key in self.prompt_graphs:
                if packed:
                    return self._graph_packed_chunk(self.prompt_graphs[key], batch, arrays, history, chunk, want_rows)
                i, first, count = chunk.pieces[0]
                return self._graph_chunk(arrays[i][first:first + count], batch[i].slot, history[i] + first, want_rows)
            record = key                      # this one runs the ordinary way (it also warms the kernels up), then the graph is made
        out = self._run_chunk_eager(batch, arrays, history, chunk, want_rows)
        if record is not None:
            if record[3]:
                self._record_packed_chunk(record[0], record[1], record[2])
            else:
                self._record_chunk(record[0], record[1], record[2])
        return out

    # ---- full chunks that hold pieces of several sequences ----
    def _packed_layout(self, n: int, n_want: int) -> Dict[str, Tuple[int, int]]:
        """Where the parts of a packed chunk's description lie in its input buffer: name -> (offset, length).  The
        sequence axis has room for MAX_GRAPH_PIECES pieces and one sequence more that is always empty (the query tiles
        that a chunk does not fill point at it); the tile axis has room for every piece's last, partial tile."""
        seqs = MAX_GRAPH_PIECES + 1
        tiles = n // PREFILL_TILE_ROWS + MAX_GRAPH_PIECES
        layout, at = {}, 0
        for name, length in (("ids", n), ("positions", n), ("token_seq", n), ("cu_q", seqs + 1), ("kv_len", seqs), ("slot", seqs),
                             ("want", n_want), ("tile_seq", tiles), ("tile_row", tiles)):
            layout[name] = (at, length)
            at += length
        layout["total"] = (0, at)
        return layout

    def _record_packed_chunk(self, n: int, n_want: int, bound: int) -> None:
        """Records the graph of a full chunk of ``n`` tokens from several sequences.  Nothing runs."""
        ops, dev = self.ops, self.ops.device
        lay = self._packed_layout(n, n_want)
        inputs = torch.zeros(lay["total"][1], dtype=torch.int32, device=dev)
        g = _PromptGraph(inputs, inputs[:0])

        def part(name: str) -> torch.Tensor:
            o, length = lay[name]
            return inputs[o:o + length]

        def body():
            ws = ops.workspace
            if ws is not None:
                ws.require(n, MAX_GRAPH_PIECES + 1)
            ops.begin_step()
            ctx = StepContext(
                n_tokens=n, n_seqs=MAX_GRAPH_PIECES + 1, is_decode=False, captured=True, q_lens=[n], kv_lens=[], slots=[],
                max_q_len=n, max_kv_len=bound, token_ids=part("ids"), positions=part("positions"), token_seq=part("token_seq"),
                cu_q=part("cu_q"), kv_len_dev=part("kv_len"), slot_dev=part("slot"), cache=self.cache)
            ctx.q_tiles = (part("tile_seq"), part("tile_row"), lay["tile_seq"][1])
            ctx.extras["step_begun"] = True
            return self.model.forward(ctx, part("want") if n_want else None)

        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            g.logits = body()
        g.graph = graph
        self.prompt_graphs[(n, n_want, bound, True)] = g

    def _graph_packed_chunk(self, g: "_PromptGraph", batch, arrays, history, chunk: Chunk, want_rows: List[int]) -> Optional[torch.Tensor]:
        n = self.chunk_tokens
        lay = self._packed_layout(n, len(want_rows))
        host = np.zeros(lay["total"][1], dtype=np.int32)
        seqs = MAX_GRAPH_PIECES + 1
        cu_q = np.full(seqs + 1, n, dtype=np.int32)          # sequences behind the chunk's pieces: no tokens, no keys
        kv_len = np.zeros(seqs, dtype=np.int32)
        slot = np.full(seqs, batch[chunk.pieces[0][0]].slot, dtype=np.int32)
        at = 0
        tile_seq, tile_row = [], []
        for k, (i, first, count) in enumerate(chunk.pieces):
            start = history[i] + first
            o = lay["ids"][0] + at
            host[o:o + count] = arrays[i][first:first + count]
            o = lay["positions"][0] + at
            host[o:o + count] = np.arange(start, start + count, dtype=np.int32)
            o = lay["token_seq"][0] + at
            host[o:o + count] = k
            cu_q[k] = at
            kv_len[k] = start + count
            slot[k] = batch[i].slot
            rows = np.arange(0, count, PREFILL_TILE_ROWS, dtype=np.int32)
            tile_seq.append(np.full(rows.shape[0], k, dtype=np.int32))
            tile_row.append(rows)
            at += count
        n_tiles = lay["tile_seq"][1]
        ts = np.full(n_tiles, seqs - 1, dtype=np.int32)       # unused tiles belong to the empty sequence
        tr = np.zeros(n_tiles, dtype=np.int32)
        used = np.concatenate(tile_seq)
        ts[:used.shape[0]] = used
        tr[:used.shape[0]] = np.concatenate(tile_row)
        for name, values in (("cu_q", cu_q), ("kv_len", kv_len), ("slot", slot), ("want", np.asarray(want_rows, dtype=np.int32)),
                             ("tile_seq", ts), ("tile_row", tr)):
            o, length = lay[name]
            host[o:o + length] = values
        g.inputs.copy_(torch.from_numpy(host))
        g.graph.replay()
        return None if g.logits is None else g.logits.clone()

    def _run_chunk_eager(self, batch, arrays, history, chunk: Chunk, want_rows: List[int]) -> Optional[torch.Tensor]:
        kv_lens: List[int] = []
        q_lens: List[int] = []
        slots: List[int] = []
        id_parts, pos_parts = [], []
        for i, first, count in chunk.pieces:
            start = history[i] + first
            id_parts.append(arrays[i][first:first + count])
            pos_parts.append(np.arange(start, start + count, dtype=np.int32))
            kv_lens.append(start + count)
            q_lens.append(count)
            slots.append(batch[i].slot)
        ids = np.concatenate(id_parts)
        q_arr = np.asarray(q_lens, dtype=np.int32)
        cu_q = np.zeros(len(q_lens) + 1, dtype=np.int32)
        np.cumsum(q_arr, out=cu_q[1:])
        n_tok, n_seq = int(ids.shape[0]), len(slots)
        ws = self.ops.workspace
        if ws is not None:
            ws.require(n_tok, n_seq)          # a step the workspace was not sized for is refused before anything runs
        self.ops.begin_step()
        # query tiles of the prefill attention kernel: (sequence, first token of the tile)
        tiles_per = (q_arr + PREFILL_TILE_ROWS - 1) // PREFILL_TILE_ROWS
        tile_seq = np.repeat(np.arange(len(q_lens), dtype=np.int32), tiles_per)
        tile_first = np.zeros(len(q_lens), dtype=np.int32)
        np.cumsum(tiles_per[:-1], out=tile_first[1:])
        tile_row = (np.arange(int(tiles_per.sum()), dtype=np.int32) - np.repeat(tile_first, tiles_per)) * PREFILL_TILE_ROWS
        packed = torch.from_numpy(np.concatenate([
            ids, np.concatenate(pos_parts), np.repeat(np.arange(len(q_lens), dtype=np.int32), q_arr), cu_q,
            np.asarray(kv_lens, dtype=np.int32), np.asarray(slots, dtype=np.int32), np.asarray(want_rows, dtype=np.int32),
            tile_seq, tile_row.astype(np.int32)]).astype(np.int32, copy=False))
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
        ctx.q_tiles = (cut(len(tile_seq)), cut(len(tile_row)), len(tile_seq))
        ctx.extras["step_begun"] = True
        if self.taps is not None:
            ctx.extras["taps"] = self.taps
        return self.model.forward(ctx, rows)
