"""One allocation with named regions: weights, the step workspace, per-sequence state and
the key-value pages.

The reference takes a fraction of the device's memory with one ``cudaMalloc``, hands weights
out from the front, places a step's activations at fixed offsets that alias one another
across layers, and gives the rest to the cache (src/model/memory.cuh:22-115,
src/model/model.cuh:103-120, src/model/kvcache.cuh:47-64); when a request does not fit it
prints a line and returns a null pointer (memory.cuh:92-96).  Here the same layout is a
table of regions over one tensor of bytes, and a request that does not fit raises
:class:`PoolExhausted`, which names the region.

An arena without a device (``device=None``) hands out tensors without storage ("meta"
tensors) and only counts: that is how the workspace is sized, by running the model's own
forward pass once on such tensors (see cpmcu_b200.ops.dry).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

import os

ALIGN = int(os.environ.get("CPMCU_ARENA_ALIGN", "256"))      # every tensor of the arena starts at a multiple of this


def round_up(n: int, to: int = ALIGN) -> int:
    return (int(n) + to - 1) // to * to


def nbytes_of(shape: Sequence[int], dtype: torch.dtype) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty((), dtype=dtype).element_size()


class PoolExhausted(MemoryError):
    """A region of the arena (or the arena itself) cannot hold what was asked of it."""

    def __init__(self, region: str, wanted: int, capacity: int, used: int = 0, what: str = "", unit: str = "bytes"):
        self.region, self.wanted, self.capacity, self.used = region, int(wanted), int(capacity), int(used)
        msg = (f"memory pool exhausted in region '{region}': {self.wanted:,} {unit} wanted, "
               f"{self.capacity - self.used:,} of {self.capacity:,} free")
        if what:
            msg += f" ({what})"
        super().__init__(msg)


class Region:
    """A contiguous piece of the arena with a bump pointer.  ``size`` None = unbounded (counting only)."""

    def __init__(self, arena: "Arena", name: str, offset: int, size: Optional[int]):
        self.arena, self.name, self.offset, self.size = arena, name, int(offset), size
        self.used = 0
        self.peak = 0

    def reset(self, mark: int = 0) -> None:
        self.used = mark

    def take(self, nbytes: int, what: str = "") -> int:
        """Offset (in the arena) of ``nbytes`` fresh bytes."""
        start = round_up(self.used)
        end = start + int(nbytes)
        if self.size is not None and end > self.size:
            raise PoolExhausted(self.name, nbytes, self.size, self.used, what)
        self.used = end
        self.peak = max(self.peak, end)
        return self.offset + start

    def tensor(self, shape: Sequence[int], dtype: torch.dtype, zero: bool = False, what: str = "") -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        n = nbytes_of(shape, dtype)
        at = self.take(n, what)
        return self.arena.view(at, n, shape, dtype, zero)


class Arena:
    GUARD_BYTE = 0xA5

    def __init__(self, total_bytes: Optional[int], device: "torch.device | str | None", guards: bool = False):
        """``device`` None: a counting arena without memory (``total_bytes`` may be None = unbounded).
        ``guards``: every region is followed by ALIGN bytes of a fixed pattern that nothing may write;
        ``check_guards`` says which region was overrun (for checked runs; ``total_bytes`` must leave room for them)."""
        self.guards = bool(guards)
        self.guard_at: Dict[str, int] = {}
        self.total = None if total_bytes is None else int(total_bytes)
        self.device = None if device is None else torch.device(device)
        self.buffer: Optional[torch.Tensor] = None
        if self.device is not None:
            if self.total is None:
                raise ValueError("an arena with memory needs a size")
            try:
                raw = torch.empty(self.total + ALIGN, dtype=torch.uint8, device=self.device)
            except RuntimeError as e:          # torch's out-of-memory error
                raise PoolExhausted("arena", self.total, 0, 0, f"the device could not give one piece of this size: "
                                    f"{str(e).splitlines()[0][:120]}") from None
            skip = (-raw.data_ptr()) % ALIGN   # offsets inside the arena are multiples of ALIGN: so are the addresses
            self.buffer = raw[skip:skip + self.total]
        self.regions: Dict[str, Region] = {}
        self.carved = 0

    def carve(self, name: str, nbytes: Optional[int]) -> Region:
        """The next region, ``nbytes`` long (None: unbounded, in a counting arena only)."""
        if name in self.regions:
            raise ValueError(f"region '{name}' exists already")
        if nbytes is None:
            if self.buffer is not None:
                raise ValueError("only a counting arena has unbounded regions")
            region = Region(self, name, 0, None)
        else:
            size = round_up(nbytes)
            if self.total is not None and self.carved + size > self.total:
                raise PoolExhausted("arena", size, self.total, self.carved, f"carving region '{name}'")
            region = Region(self, name, self.carved, size)
            self.carved += size
            if self.guards and self.buffer is not None:
                if self.carved + ALIGN > self.total:
                    raise PoolExhausted("arena", ALIGN, self.total, self.carved, f"the guard behind region '{name}'")
                self.guard_at[name] = self.carved
                self.buffer[self.carved:self.carved + ALIGN].fill_(self.GUARD_BYTE)
                self.carved += ALIGN
        self.regions[name] = region
        return region

    def check_guards(self) -> None:
        """Raises if the bytes behind a region have been written (something ran over the region's end)."""
        for name, at in self.guard_at.items():
            g = self.buffer[at:at + ALIGN]
            if not bool((g == self.GUARD_BYTE).all()):
                first = int((g != self.GUARD_BYTE).nonzero()[0])
                raise RuntimeError(f"memory arena: the guard behind region '{name}' was overwritten "
                                   f"(first at byte {first} past the region's end)")

    def view(self, at: int, nbytes: int, shape: Tuple[int, ...], dtype: torch.dtype, zero: bool) -> torch.Tensor:
        if self.buffer is None:
            return torch.empty(shape, dtype=dtype, device="meta")
        t = self.buffer[at:at + nbytes].view(dtype).view(shape)
        if zero:
            t.zero_()
        return t

    def report(self) -> Dict[str, Tuple[int, int]]:
        """region -> (bytes it has, most bytes it ever held)."""
        return {name: (r.size if r.size is not None else r.peak, r.peak) for name, r in self.regions.items()}


class Workspace:
    """The memory of one step: a persistent part (token descriptors, the residual stream, what outlives
    a layer) and two frames that the layers use in turn.

    A layer's intermediates live in the frame of its parity and die when the layer after next begins;
    the one tensor that crosses a layer boundary (the feed-forward's output, whose addition the next
    layer's norm performs) is still intact then, because the next layer writes into the other frame.
    This is the table of lifetimes that the reference writes as explicit offsets
    (src/model/model.cuh:103-120, src/model/layer.cuh:30-35).
    """

    def __init__(self, persistent: Region, frames: Sequence[Region], sized_tokens: int = 0, sized_seqs: int = 0):
        self.persistent = persistent
        self.frames = list(frames)
        self.current = persistent
        self.sized_tokens, self.sized_seqs = int(sized_tokens), int(sized_seqs)

    def begin_step(self) -> None:
        self.persistent.reset()
        for f in self.frames:
            f.reset()
        self.current = self.persistent

    def begin_layer(self, k: int) -> None:
        self.current = self.frames[k % len(self.frames)]
        self.current.reset()

    def end_layers(self) -> None:
        self.current = self.persistent

    def alloc(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        return self.current.tensor(shape, dtype, what="a step's intermediate tensor")

    def require(self, n_tokens: int, n_seqs: int) -> None:
        """Refuses, before anything runs, a step larger than the workspace was sized for."""
        if self.sized_tokens and n_tokens > self.sized_tokens:
            raise PoolExhausted("workspace", n_tokens, self.sized_tokens, 0,
                                f"a step of {n_tokens} tokens; the workspace was sized for {self.sized_tokens} tokens a step", "tokens")
        if self.sized_seqs and n_seqs > self.sized_seqs:
            raise PoolExhausted("workspace", n_seqs, self.sized_seqs, 0,
                                f"a step of {n_seqs} sequences; the workspace was sized for {self.sized_seqs}", "sequences")

    def peaks(self) -> Tuple[int, int]:
        """(most bytes the persistent part held, most bytes a frame held)."""
        return self.persistent.peak, max((f.peak for f in self.frames), default=0)


def plan_storage(budget: Optional[int], weight_bytes: int, workspace_bytes: int, cache_bytes_of, max_tokens: Optional[int],
                 page_tokens: int = 64) -> Tuple[int, int]:
    """How many tokens the cache holds and how large the arena is: (tokens, total bytes).

    ``cache_bytes_of(tokens)`` gives the bytes of page tables, per-sequence state and pages of a cache for that
    many tokens.  With ``max_tokens`` the cache is made for exactly that many (rounded down to whole pages) and
    the arena is as large as that takes; ``budget``, if given, must cover it.  Without ``max_tokens`` the cache
    takes what ``budget`` leaves after weights and workspace.  Raises :class:`PoolExhausted` naming what did not fit."""
    fixed = round_up(weight_bytes) + round_up(workspace_bytes)
    slack = 64 * ALIGN                                     # alignment gaps between a region's tensors
    if max_tokens is not None:
        tokens = max(page_tokens, int(max_tokens) // page_tokens * page_tokens)
        total = fixed + round_up(cache_bytes_of(tokens)) + slack
        if budget is not None and total > budget:
            raise PoolExhausted("arena", total, budget, 0, f"weights {weight_bytes:,} + workspace {workspace_bytes:,} + a cache "
                                f"of {tokens} tokens do not fit the memory limit")
        return tokens, total
    if budget is None:
        raise ValueError("plan_storage needs a budget or max_tokens")
    if fixed + slack >= budget:
        raise PoolExhausted("weights" if round_up(weight_bytes) >= budget else "workspace", fixed, budget, 0,
                            f"weights {weight_bytes:,} + workspace {workspace_bytes:,} bytes leave nothing of the memory limit")
    room = budget - fixed - slack
    per_token = max(1, cache_bytes_of(2 * page_tokens) - cache_bytes_of(page_tokens)) // page_tokens
    tokens = room // per_token // page_tokens * page_tokens
    for _ in range(8):                                     # page tables grow with the cache: step down until it fits
        if tokens < 2 * page_tokens:
            raise PoolExhausted("cache", cache_bytes_of(2 * page_tokens), room, 0,
                                "the memory limit leaves no room for a cache of two pages")
        need = cache_bytes_of(tokens)
        if need <= room:
            return tokens, budget
        tokens -= ((need - room) // per_token // page_tokens + 1) * page_tokens
    raise PoolExhausted("cache", cache_bytes_of(max(tokens, page_tokens)), room, 0, "no cache size fits the memory limit")
