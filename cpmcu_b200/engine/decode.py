"""Decode steps that run without the host in between: one token per live sequence,
sampled on the device and fed back as the next input, optionally as a CUDA graph.

The batch lives in fixed device buffers (ids, positions, key counts, slots, random
keys); a step reads them, runs the model on one token per entry, samples, and
advances the buffers.  The buffers have a bucket size (a power of two); entries
beyond the live sequences are padding that points at a scratch sequence and never
advances, so padding changes no result.  One graph is captured per bucket size and
replayed whatever the sequences' lengths are, because every kernel reads lengths and
pages from device memory.  The reference captures its decode graph anew whenever the
padded length or the token count changes (src/entry.cu:562-584) and returns to the host
for every token (cpmcu/llm.py:361-373).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import StepContext
from ..sampling import SamplingParams
from .step import Stepper


def bucket_size(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class _Bucket:
    def __init__(self, size: int, device: torch.device):
        i32 = dict(dtype=torch.int32, device=device)
        self.size = size
        self.ids = torch.zeros(size, **i32)
        self.positions = torch.zeros(size, **i32)
        self.kv_len = torch.ones(size, **i32)
        self.slot = torch.zeros(size, **i32)
        self.token_seq = torch.arange(size, **i32)
        self.cu_q = torch.arange(size + 1, **i32)
        self.want_rows = torch.arange(size, **i32)
        self.live = torch.zeros(size, **i32)
        self.seq_key = torch.zeros(size, **i32)
        self.step_key = torch.zeros(size, **i32)
        self.temperature = torch.zeros(size, dtype=torch.float32, device=device)
        self.top_p = torch.ones(size, dtype=torch.float32, device=device)
        self.sampled = torch.zeros(size, **i32)
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.warm = False
        self.launches = 0           # kernels of this library in one step


class DecodeRunner:
    def __init__(self, stepper: Stepper, use_graph: bool = True, seed: int = 0):
        self.stepper = stepper
        self.model = stepper.model
        self.cache = stepper.cache
        self.ops = stepper.ops
        self.use_graph = bool(use_graph)
        self.seed = int(seed)
        self.buckets: Dict[int, _Bucket] = {}
        self.pad_slot = self.cache.open_sequence()       # scratch sequence the padding entries use
        self.cache.reserve(self.pad_slot, 1)
        self.cache.set_length(self.pad_slot, 1)
        self.cache.sync()
        self.current: Optional[_Bucket] = None
        self.slots: List[int] = []
        self.pinned = None
        self.pinned_in = None
        self.feed_done = None

    # ---- one step's work on the device ----
    def _body(self, b: _Bucket, captured: bool, slots: Sequence[int] = ()) -> None:
        """One step on the bucket's buffers.  Captured: the host lists of the context are empty and the longest
        sequence is given as the cache's capacity, because the same recording runs for any lengths.  Not captured:
        the host lists describe the live sequences (``slots``) followed by the padding entries, as the step
        function's do, so a part that decides on the host works here too."""
        if captured:
            kv_lens, slot_list, longest = [], [], self.cache.max_pages_per_seq * 64
        else:
            pad = b.size - len(slots)
            kv_lens = [self.cache.length(s) + 1 for s in slots] + [1] * pad
            slot_list = list(slots) + [self.pad_slot] * pad
            longest = max(kv_lens)
        ctx = StepContext(
            n_tokens=b.size, n_seqs=b.size, is_decode=True, captured=captured,
            q_lens=[1] * b.size, kv_lens=kv_lens, slots=slot_list, max_q_len=1, max_kv_len=longest,
            token_ids=b.ids, positions=b.positions, token_seq=b.token_seq, cu_q=b.cu_q,
            kv_len_dev=b.kv_len, slot_dev=b.slot, cache=self.cache,
        )
        if not captured and self.stepper.taps is not None:
            ctx.extras["taps"] = self.stepper.taps
        ws = self.ops.workspace
        if ws is not None:
            ws.require(b.size, b.size)
        self.ops.begin_step()
        ctx.extras["step_begun"] = True
        b.logits = self.model.forward(ctx, b.want_rows)
        self.ops.sample(b.logits, b.temperature, b.top_p, self.seed, b.seq_key, b.step_key, out=b.sampled)
        self.ops.advance_decode(b.ids, b.positions, b.kv_len, b.step_key, b.sampled, b.live)

    def _bucket(self, n: int) -> _Bucket:
        size = bucket_size(n)
        b = self.buckets.get(size)
        if b is None:
            b = _Bucket(size, self.ops.device)
            b.slot.fill_(self.pad_slot)
            self.buckets[size] = b
        return b

    def _prepare(self, b: _Bucket) -> None:
        """Warm-up and capture happen on padding only, so they touch no sequence."""
        if b.warm:
            return
        b.slot.fill_(self.pad_slot)
        b.live.zero_()
        b.positions.zero_()
        b.kv_len.fill_(1)
        b.ids.zero_()
        b.temperature.zero_()
        torch.cuda.synchronize()
        from ..ops import library
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        before = library.LAUNCHES[0]
        with torch.cuda.stream(side):
            self._body(b, captured=self.use_graph)
        b.launches = library.LAUNCHES[0] - before
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self.use_graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._body(b, captured=True)
            b.graph = g
        b.warm = True

    # ---- batches ----
    def start(self, slots: Sequence[int], last_tokens: Sequence[int], seq_keys: Sequence[int],
              step_keys: Sequence[int], sampling: Sequence[SamplingParams]) -> None:
        """Sets the batch: ``last_tokens`` are the tokens to feed next; every sequence's
        position is its current length in the cache."""
        n = len(slots)
        b = self._bucket(n)
        self._prepare(b)
        pad = b.size - n
        lengths = [self.cache.length(s) for s in slots]
        host = torch.tensor(
            list(last_tokens) + [0] * pad + lengths + [0] * pad + [l + 1 for l in lengths] + [1] * pad
            + list(slots) + [self.pad_slot] * pad + [1] * n + [0] * pad + list(seq_keys) + [0] * pad
            + list(step_keys) + [0] * pad, dtype=torch.int32).view(7, b.size).to(self.ops.device)
        b.ids.copy_(host[0]); b.positions.copy_(host[1]); b.kv_len.copy_(host[2]); b.slot.copy_(host[3])
        b.live.copy_(host[4]); b.seq_key.copy_(host[5]); b.step_key.copy_(host[6])
        fl = torch.tensor([p.temperature for p in sampling] + [0.0] * pad + [p.top_p for p in sampling] + [1.0] * pad,
                          dtype=torch.float32).view(2, b.size).to(self.ops.device)
        b.temperature.copy_(fl[0]); b.top_p.copy_(fl[1])
        self.current = b
        self.slots = list(slots)

    def feed(self, tokens: Sequence[int]) -> None:
        """The next step's input tokens from the host (pinned memory, asynchronous copy).  Without
        this call a step feeds on the tokens the last step sampled, which are already on the device."""
        n = len(tokens)
        if self.pinned_in is None or self.pinned_in.numel() < self.current.size:
            self.pinned_in = torch.empty(max(64, self.current.size), dtype=torch.int32).pin_memory()
            self.pinned_in_np = self.pinned_in.numpy()          # the same memory, written without building a tensor
            self.feed_done = torch.cuda.Event()
        else:
            self.feed_done.synchronize()        # the last copy out of the pinned buffer must be over before it is rewritten
        self.pinned_in_np[:n] = tokens
        self.current.ids[:n].copy_(self.pinned_in[:n], non_blocking=True)
        self.feed_done.record()

    def step(self) -> torch.Tensor:
        """Runs one decode step of the current batch; returns the sampled tokens (device,
        int32, one per live sequence; valid until the next step)."""
        b = self.current
        if self.cache.grow_by_one(self.slots):
            self.cache.sync()
        if b.graph is not None:
            b.graph.replay()
        else:
            self._body(b, captured=False, slots=self.slots)
        self.cache.grown_by_one(self.slots)
        return b.sampled[:len(self.slots)]

    @property
    def launches_per_graph(self) -> int:
        return self.current.launches if self.current is not None else 0

    def logits(self) -> torch.Tensor:
        """fp32 logits of the last step, one row per live sequence."""
        return self.current.logits[:len(self.slots)]

    def read_tokens(self) -> List[int]:
        """The last step's sampled tokens on the host (waits for the step)."""
        n = len(self.slots)
        if self.pinned is None or self.pinned.numel() < self.current.size:
            self.pinned = torch.empty(max(64, self.current.size), dtype=torch.int32).pin_memory()
            self.pinned_np = self.pinned.numpy()
            self.read_done = torch.cuda.Event()
        self.pinned[:n].copy_(self.current.sampled[:n], non_blocking=True)
        self.read_done.record()
        self.read_done.synchronize()
        return self.pinned_np[:n].tolist()
