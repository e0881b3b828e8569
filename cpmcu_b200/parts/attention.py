"""Grouped-query attention over the paged cache.

One product gives q, k and v of a token (the reference keeps Wq, Wk, Wv in one
buffer for the same reason, src/model/attn.cuh:113-118, 235-243); queries and keys
are rotated and keys and values stored into the cache in one kernel; attention
runs over the cache, which then already holds this step's tokens; the output
projection follows (src/model/attn.cuh:185-229).  With ``sparse`` given, queries that
see more than ``dense_len`` keys attend only to selected key blocks (InfLLM-v2,
src/model/minicpm4/minicpm4_attn.cuh:95-202); that rule is per query, so it does not
depend on how tokens are cut into steps.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Mapping, Optional

import torch

from .base import MIXERS, POSITIONS, CacheNeeds, Mixer, PartSpec, WeightSpec, build_part


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    @property
    def recordable_prompt(self) -> bool:
        return bool(self.position.recordable_prompt)

    def __init__(self, ops, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PartSpec, window: Optional[int] = None, sparse: Optional[Mapping[str, int]] = None,
                 softmax_scale: Optional[float] = None, position_name: str = ""):
        """``position_name``: infix of the position part's own tensors below this part's prefix (an encoding with
        learned tables declares them in its ``weight_specs``; the rotary encodings have none)."""
        super().__init__(ops)
        if window and sparse:
            # a windowed lane gives pages back that the block selection (leading blocks, chosen far blocks, the
            # scores over all pooled keys) would still follow
            raise ValueError("gqa_attention takes a window or a sparse configuration, not both")
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot be grouped over {n_kv_heads} key-value heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
        self.hidden_size, self.n_heads, self.n_kv, self.d = int(hidden_size), int(n_heads), int(n_kv_heads), int(head_dim)
        self.window = int(window) if window else 0
        self.sparse = dict(sparse) if sparse else None
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.d)
        self.position = build_part(POSITIONS, position, ops)
        self.position_name = str(position_name)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    # ---- weights ----
    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, d = self.hidden_size, self.d
        specs = {
            "q_proj.weight": WeightSpec((self.n_heads * d, h)),
            "k_proj.weight": WeightSpec((self.n_kv * d, h)),
            "v_proj.weight": WeightSpec((self.n_kv * d, h)),
            "o_proj.weight": WeightSpec((h, self.n_heads * d)),
        }
        for name, spec in self.position.weight_specs().items():
            specs[self.position_name + name] = spec
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        own = self.position.weight_specs()
        if own:
            self.position.load_weights({n: tensors[self.position_name + n] for n in own})
        self.w_qkv = self.ops.keep(torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]],
                                             dim=0).contiguous())
        self.w_o = self.ops.keep(tensors["o_proj.weight"].contiguous())

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    # ---- cache ----
    def cache_needs(self) -> CacheNeeds:
        stride = self.sparse["kernel_stride"] if self.sparse else 0
        kernel = self.sparse["kernel_size"] if self.sparse else 0
        return CacheNeeds(kv_heads=self.n_kv, head_dim=self.d, window=self.window or None,
                          pooled_stride=stride, pooled_kernel=kernel)

    def cache_bytes_read(self, kv_len: int) -> int:
        keys = min(kv_len, self.window) if self.window else kv_len
        pooled = 0
        if self.sparse is not None and kv_len > self.sparse.get("dense_len", 0):
            # the leading and chosen blocks (topk of them) and the local window, and every visible pooled key (fp32)
            sp = self.sparse
            blocks = sp["topk"] + sp["window_size"] // sp["block_size"]
            keys = min(kv_len, blocks * sp["block_size"])
            pooled = max(0, (kv_len - sp["kernel_size"]) // sp["kernel_stride"] + 1) * self.n_kv * self.d * 4
        return 2 * keys * self.n_kv * self.d * self.ops.element_size + pooled

    # ---- forward ----
    def forward(self, ctx, y: torch.Tensor, lane, writes_cache: bool) -> torch.Tensor:
        ops = self.ops
        if lane.k is not None:
            ops.set_page_limit(lane.k.shape[0])          # the checked build's kernels compare page numbers with it
        qkv = ops.linear(y, self.w_qkv)
        inv_freq, magnitude, rot_dim = self.position.rotary() or (None, 1.0, -1)
        k_cache, v_cache = lane.k, lane.v
        if rot_dim < 0:
            # an encoding that is not a rotation of pairs transforms q and k itself
            row = qkv.view(ctx.n_tokens, self.n_heads + 2 * self.n_kv, self.d)
            self.position.apply(ctx, row[:, :self.n_heads], row[:, self.n_heads:self.n_heads + self.n_kv])
            inv_freq, magnitude, rot_dim = None, 1.0, 0
        if rot_dim >= 0 and ops.fused_decode_ok(ctx, self.d, rot_dim, self.window, self.sparse):
            # one token per sequence: the attention kernel rotates, stores the new key and value, and attends
            out = ops.decode_attention_rope(qkv, lane, ctx.kv_len_dev, ctx.slot_dev, self.n_heads, self.n_kv, self.d,
                                            self.scale, inv_freq if rot_dim else None, magnitude, writes_cache)
            return ops.linear(out, self.w_o)
        q = ops.rope_store(qkv, self.n_heads, self.n_kv, self.d, ctx.positions, ctx.token_seq, ctx.slot_dev,
                           lane.page_table, k_cache if writes_cache else None, v_cache if writes_cache else None,
                           inv_freq, magnitude, rot_dim)
        block_list, block_size = None, 0
        if self.sparse is not None:
            if writes_cache:
                ops.pool_keys(ctx, lane, self.n_kv, self.d, self.sparse["kernel_size"], self.sparse["kernel_stride"])
            if ctx.max_kv_len > self.sparse.get("dense_len", 0):      # in a recorded step an upper bound: still the right test
                block_list, block_size = ops.select_blocks(ctx, q, lane, self.n_kv, self.scale, self.sparse)
                taps = ctx.extras.get("taps")
                if taps is not None and not ctx.captured:
                    # a caller that wants to see the choice (tests do): lane, the step's slots, and per token its
                    # sequence, position and block lists
                    taps.setdefault("block_lists", []).append(
                        (lane.index, list(ctx.slots), ctx.token_seq.clone(), ctx.positions.clone(), block_list.clone()))
        out = ops.attention(ctx, q, lane, self.n_kv, self.scale, self.window, block_list, block_size)
        return ops.linear(out, self.w_o)
