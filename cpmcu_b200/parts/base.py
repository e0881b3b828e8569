"""Interfaces of the parts a model is put together from, and their registries.

A model is data: a :class:`ModelSpec` lists layers, each layer names its mixer, its
feed-forward, its norms and how they are arranged in a block, every one with its
sizes and constants as parameters; a schedule lists the order in which layers run.
Parts are looked up by name in the registries below, so a new mixer, feed-forward,
norm, position encoding or block arrangement is one class and one ``register``
call; no part knows which model it belongs to.

The reference builds its layers from fixed classes (src/model/layer.cuh:10-45,
src/model/attn.cuh:58-160, src/model/ffn.cuh:18-60); this file is the seam that
replaces that fixed structure.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Generic, List, Mapping, Optional, Sequence, Tuple, Type, TypeVar

import torch

T = TypeVar("T")

# Tokens per page of the key-value cache.  The one Python-side definition (cache and kernel wrappers import it); the
# kernels' own constant (csrc/common.cuh) is compared with it when the library is loaded.
PAGE_TOKENS = 64
# Query tokens per tile of the tiled prompt attention kernels (StepContext.q_tiles is made for this size).
QUERY_TILE_TOKENS = 64


class Registry(Generic[T]):
    """A table from a name to a class, with an error that lists what is known."""

    def __init__(self, what: str):
        self.what = what
        self._table: Dict[str, T] = {}

    def register(self, name: str) -> Callable[[T], T]:
        def deco(obj: T) -> T:
            if name in self._table and self._table[name] is not obj:
                raise KeyError(f"{self.what} '{name}' is already registered")
            self._table[name] = obj
            return obj
        return deco

    def unregister(self, name: str) -> None:
        self._table.pop(name, None)

    def get(self, name: str) -> T:
        try:
            return self._table[name]
        except KeyError:
            raise KeyError(f"unknown {self.what} '{name}'; known: {sorted(self._table)}") from None

    def names(self) -> List[str]:
        return sorted(self._table)

    def __contains__(self, name: str) -> bool:
        return name in self._table


# ---------------------------------------------------------------------------
# specifications (plain data)
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class PartSpec:
    """Which part (a registry name) and its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block) of a mixer, a feed-forward and their norms.

    ``prefix`` is the layer's part of the tensor names ("model.layers.3."); the
    names below it are given by ``names``: sub-part -> infix ("self_attn." ...).
    ``feed_forward`` and ``feed_forward_norm`` may be None: a layer of a mixer alone.
    """

    block: PartSpec
    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    mixer_norm: PartSpec
    feed_forward_norm: Optional[PartSpec]
    prefix: str
    names: Mapping[str, str]


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``lane`` is the cache lane (keys, values, state) the run
    uses; ``writes_cache`` is False when the run only reads a lane an earlier run
    of this step has written (a layer that shares another layer's keys and values)."""

    layer: int
    lane: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Sequence[LayerSpec]
    schedule: Sequence[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    embedding_name: str = "model.embed_tokens."
    final_norm_name: str = "model.norm."
    head_name: str = "lm_head."
    stop_token_ids: Sequence[int] = ()
    max_positions: int = 0

    def n_lanes(self) -> int:
        return 1 + max(e.lane for e in self.schedule)


def default_schedule(n_layers: int) -> List[ScheduleEntry]:
    return [ScheduleEntry(layer=i, lane=i, writes_cache=True) for i in range(n_layers)]


@dataclass(frozen=True)
class WeightSpec:
    """Shape and role of one tensor.

    role "matrix": an operand of a matrix product or a lookup table of rows; held in
    the compute dtype.  role "vector": norm weights and other small tensors; a tensor
    stored in 32-bit stays in 32-bit.  role "table": integers, held as int32.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeeds:
    """What one cache lane must hold for every sequence.

    kv_heads/head_dim: one key row and one value row per token and key-value head
    (0 heads = none).  window: None if every key stays needed, else the number of
    most recent tokens that do.  pooled_stride/pooled_kernel: an extra row per
    ``pooled_stride`` tokens (mean-pooled keys); 0 = none.  state: tensors of fixed
    size per sequence, name -> (shape, dtype); they are zero when a sequence starts.
    """

    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    pooled_stride: int = 0
    pooled_kernel: int = 0
    state: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]] = field(default_factory=dict)

    def group_key(self) -> Tuple:
        return (self.kv_heads, self.head_dim, self.window, self.pooled_stride, self.pooled_kernel)


# ---------------------------------------------------------------------------
# part interfaces
# ---------------------------------------------------------------------------

class Part:
    """Common to all parts: declared weights, and loading them.

    ``ops`` is the kernel library bound to a compute dtype (see cpmcu_b200.ops); a
    part calls kernels only through it.
    """

    def __init__(self, ops):
        self.ops = ops

    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Tensor names below this part's prefix -> shape and role."""
        return {}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives exactly the tensors of ``weight_specs`` (already on the device)."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads (each tensor once)."""
        return 0

    # True if ``forward`` reads nothing of the batch on the host but ``n_tokens``, ``n_seqs``, ``q_lens`` and the
    # upper bound ``max_kv_len``, for prompts too: such a part can be recorded into a graph for a prompt chunk
    # (a part that walks ``ctx.slots`` or ``ctx.kv_lens`` on the host cannot; the default is the safe answer).
    recordable_prompt = False


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: fp32 [tokens, hidden] residual stream -> normed [tokens or len(rows), hidden] in compute dtype."""
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor, scale: float,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x += scale*delta (written back unless ``rows`` is given), then forward."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information for a mixer.

    A rotary encoding that the fused rotate-and-store kernel can apply returns its
    table from ``rotary()``; any other encoding returns None there and transforms
    the queries and keys itself in ``apply``.
    """

    def rotary(self) -> Optional[Tuple[torch.Tensor, float, int]]:
        """(inv_freq fp32 [rot_dim/2], magnitude factor for cos and sin, rot_dim) or None."""
        return None

    def apply(self, ctx: "StepContext", q: torch.Tensor, k: torch.Tensor) -> None:
        """In place on q [tokens, heads, d] and k [tokens, kv_heads, d] (views with strides)."""


class Mixer(Part):
    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def forward(self, ctx: "StepContext", y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        """y: normed [tokens, hidden] (compute dtype) -> [tokens, hidden]."""
        raise NotImplementedError

    def cache_bytes_read(self, kv_len: int) -> int:
        """Bytes of cache one decode step of a sequence with ``kv_len`` keys has to read."""
        return 0


class FeedForward(Part):
    def forward(self, ctx: "StepContext", y: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class ResidualStream:
    """The fp32 residual sum of a step, with the last part's output still to be added.

    The addition of a part's output is deferred so that the next norm does it in the
    same kernel (the reference fuses the add into its norm kernel too:
    src/model/norm.cuh:53-99); the sum itself is always kept and formed in 32-bit.
    """

    def __init__(self, ops, x: torch.Tensor):
        self.ops = ops
        self.x = x
        self.pending: Optional[torch.Tensor] = None
        self.pending_scale: float = 1.0

    def add(self, delta: torch.Tensor, scale: float = 1.0) -> None:
        self.flush()
        self.pending = delta
        self.pending_scale = float(scale)

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            self.ops.residual_add(self.x, self.pending, self.pending_scale)
            self.pending = None
        return self.x

    def normed(self, norm: Norm, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.pending is None:
            return norm.forward(self.x, rows)
        y = norm.add_forward(self.x, self.pending, self.pending_scale, rows)
        if rows is None:
            self.pending = None
        return y


class Block(Part):
    """An arrangement of a mixer, a feed-forward and norms around the residual stream."""

    def __init__(self, ops, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Norm,
                 feed_forward_norm: Optional[Norm], names: Mapping[str, str]):
        super().__init__(ops)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.names = dict(names)

    def sub_parts(self) -> List[Tuple[str, Part]]:
        parts = [
            (self.names.get("mixer_norm", "mixer_norm."), self.mixer_norm),
            (self.names.get("mixer", "mixer."), self.mixer),
            (self.names.get("feed_forward_norm", "feed_forward_norm."), self.feed_forward_norm),
            (self.names.get("feed_forward", "feed_forward."), self.feed_forward),
        ]
        return [(infix, part) for infix, part in parts if part is not None]      # a layer may have no feed-forward

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out: Dict[str, WeightSpec] = {}
        for infix, part in self.sub_parts():
            for name, spec in part.weight_specs().items():
                out[infix + name] = spec
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for infix, part in self.sub_parts():
            names = part.weight_specs()
            part.load_weights({n: tensors[infix + n] for n in names})

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for _, p in self.sub_parts())

    def forward(self, ctx: "StepContext", stream: ResidualStream, lane, writes_cache: bool) -> None:
        raise NotImplementedError


MIXERS: Registry[Type[Mixer]] = Registry("mixer")
FEED_FORWARDS: Registry[Type[FeedForward]] = Registry("feed-forward")
NORMS: Registry[Type[Norm]] = Registry("norm")
POSITIONS: Registry[Type[PositionEncoding]] = Registry("position encoding")
BLOCKS: Registry[Type[Block]] = Registry("block")


def build_part(registry: Registry, spec: PartSpec, ops):
    cls = registry.get(spec.kind)
    try:
        return cls(ops, **dict(spec.params))
    except TypeError as e:
        raise TypeError(f"{registry.what} '{spec.kind}': bad parameters {sorted(spec.params)} ({e})") from None


def build_block(spec: LayerSpec, ops) -> Block:
    cls = BLOCKS.get(spec.block.kind)
    return cls(
        ops,
        mixer=build_part(MIXERS, spec.mixer, ops),
        feed_forward=build_part(FEED_FORWARDS, spec.feed_forward, ops) if spec.feed_forward is not None else None,
        mixer_norm=build_part(NORMS, spec.mixer_norm, ops),
        feed_forward_norm=build_part(NORMS, spec.feed_forward_norm, ops) if spec.feed_forward_norm is not None else None,
        names=spec.names,
        **dict(spec.block.params),
    )


# ---------------------------------------------------------------------------
# what a step hands to the parts
# ---------------------------------------------------------------------------

@dataclass
class StepContext:
    """One step's batch, as the parts see it.

    Host-side lists describe the batch for Python-level decisions; the device
    tensors are what kernels read.  Both are filled whenever a step runs eagerly:
    by the step function, and by the decode runner without a graph (its padding
    entries appear as sequences of one key in a scratch slot).

    In a captured step (``captured`` True: a decode step, or a prompt chunk of one
    sequence when every part of the model is ``recordable_prompt``) the device tensors are fixed
    buffers whose contents change between replays; the recording is made once, on
    padding entries only, and replayed for any batch.  A part may then read only:
    ``n_tokens``, ``n_seqs`` (the bucket size), ``is_decode``, ``q_lens`` (all 1, or the chunk's size),
    ``max_q_len``, ``max_kv_len`` (the cache's capacity per sequence, an upper
    bound), the device tensors, ``cache`` and its lanes.  ``kv_lens`` and ``slots`` are
    empty; everything that depends on a sequence (its slot, its length, its state
    in ``lane.state[name][slot]``) has to be reached on the device through
    ``slot_dev`` and ``kv_len_dev``, with operations that can be recorded (no
    host read, no data-dependent shapes).
    """

    n_tokens: int
    n_seqs: int
    is_decode: bool                      # every sequence brings exactly one token
    captured: bool
    # host
    q_lens: List[int]
    kv_lens: List[int]                   # keys per sequence after this step's tokens are stored
    slots: List[int]
    max_q_len: int
    max_kv_len: int
    # device (int32)
    token_ids: torch.Tensor              # [tokens]
    positions: torch.Tensor              # [tokens]
    token_seq: torch.Tensor              # [tokens] index of the token's sequence in this batch
    cu_q: torch.Tensor                   # [seqs+1] offsets of the sequences in the token axis
    kv_len_dev: torch.Tensor             # [seqs]
    slot_dev: torch.Tensor               # [seqs]
    cache: Any = None                    # cpmcu_b200.cache.Cache
    workspace: Any = None                # per-engine scratch tensors by name
    # Query tiles for mixers that work on tiles of QUERY_TILE_TOKENS consecutive tokens of one sequence (the tiled
    # prompt attention): (tile -> sequence index int32 [tiles], tile -> first token inside the sequence's tokens of
    # this step int32 [tiles], number of tiles); None when the step's maker gives none (a mixer then falls back to
    # a kernel that needs no tiles).
    q_tiles: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None
    extras: Dict[str, Any] = field(default_factory=dict)
