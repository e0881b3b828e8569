"""The kernel library as Python calls, bound to one compute dtype.

``Ops(torch.bfloat16)`` is the serving path: bf16 activations, weights and cache,
fp32 residual stream, norms, softmax and logits.  ``Ops(torch.float32)`` is the
true 32-bit path: every tensor fp32 and every matrix product done by this
library's own fp32 FMA kernel, never by a library routine that may pick a
reduced-precision mode.

Matrix products of the bf16 path go to cuBLAS through torch, as the reference's
do through ``cublasGemmEx`` (src/model/linear.cuh:8-37), unless a hand-written
kernel of this library takes the shape.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import library
from .library import check

from ..parts.base import PAGE_TOKENS, QUERY_TILE_TOKENS

F32, BF16 = 0, 1
FAST_HEAD_DIMS = (32, 64, 96, 128)       # head sizes the tensor-core attention kernels are built for
PREFILL_TILE_ROWS = QUERY_TILE_TOKENS    # query tokens per block of the prefill attention kernel


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _current_stream() -> int:
    """Handle of the stream torch would launch on now (the raw query is an order of magnitude cheaper than
    building a Stream object for every kernel launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class Ops:
    def __init__(self, dtype: torch.dtype, device: "torch.device | str" = "cuda:0"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.code = F32 if dtype == torch.float32 else BF16
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise library.KernelLibraryError("this library runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise library.KernelLibraryError("no CUDA device is available; there is no CPU path")
        self.lib = library.load()
        if int(self.lib.cpm_page_tokens()) != PAGE_TOKENS or int(self.lib.cpm_prefill_attention_tile_rows()) != PREFILL_TILE_ROWS:
            raise library.KernelLibraryError("the kernel library was built for another page or query-tile size than the package")
        self.element_size = 4 if dtype == torch.float32 else 2
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.use_tcgen05 = os.environ.get("CPMCU_TCGEN05", "1") != "0"
        self.use_tcgen05_attention = os.environ.get("CPMCU_TCGEN05_ATTENTION", "1") != "0"
        self.use_tcgen05_listed = os.environ.get("CPMCU_TCGEN05_LISTED", "1") != "0"      # block-list attention of prompts
        self.tcgen05_pair = os.environ.get("CPMCU_TCGEN05_PAIR", "0") == "1"      # pairs of blocks on 256-row tiles
        self.workspace = None       # cpmcu_b200.memory.Workspace: where a step's intermediates live (None: torch's allocator)
        self.weights = None         # cpmcu_b200.memory.Region that holds the weights (None: torch's allocator)

    _stream = staticmethod(_current_stream)

    # ---- checks ----
    def _act(self, t: torch.Tensor, what: str) -> torch.Tensor:
        if t.dtype != self.dtype or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}: needs a contiguous {self.dtype} CUDA tensor, got {t.dtype} "
                             f"{'cuda' if t.is_cuda else 'cpu'} contiguous={t.is_contiguous()}")
        return t

    @staticmethod
    def _i32(t: torch.Tensor, what: str) -> torch.Tensor:
        if t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}: needs a contiguous int32 CUDA tensor")
        return t

    @staticmethod
    def _f32(t: torch.Tensor, what: str) -> torch.Tensor:
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}: needs a contiguous float32 CUDA tensor")
        return t

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A tensor for an intermediate of the step: from the workspace when one is attached (it is valid until the
        workspace reuses its place, at the latest when the next step begins), else from torch's allocator."""
        if self.workspace is not None:
            return self.workspace.alloc(shape, dtype or self.dtype)
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def result(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A tensor the step hands to its caller (logits, sampled tokens): never from the workspace, so that it
        stays valid after later steps."""
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def keep(self, t: torch.Tensor) -> torch.Tensor:
        """A weight for good: copied into the arena's weight region when one is attached (the copy replaces the
        tensor the loader made), else the tensor itself."""
        if self.weights is None or t.device.type == "meta":
            return t
        own = self.weights.tensor(t.shape, t.dtype, what="weights")
        own.copy_(t)
        return own

    # ---- the workspace's lifetimes (no-ops without a workspace) ----
    def begin_step(self) -> None:
        if self.workspace is not None:
            self.workspace.begin_step()

    def begin_layer(self, k: int) -> None:
        if self.workspace is not None:
            self.workspace.begin_layer(k)

    def end_layers(self) -> None:
        if self.workspace is not None:
            self.workspace.end_layers()

    # ---- rows ----
    def embed(self, ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
        """ids int32 [tokens], table [vocab, hidden] -> fp32 [tokens, hidden] = table[ids] * scale."""
        self._i32(ids, "embed ids")
        self._act(table, "embedding table")
        n, hidden = ids.numel(), table.shape[1]
        out = self.empty(n, hidden, dtype=torch.float32)
        check(self.lib.cpm_embed_rows(_ptr(ids), _ptr(table), _ptr(out), n, hidden, float(scale), self.code,
                                      self._stream()), "embed")
        return out

    def add_rmsnorm(self, x: torch.Tensor, delta: Optional[torch.Tensor], alpha: float, weight: torch.Tensor,
                    eps: float, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x fp32 [tokens, hidden] (+= alpha*delta, written back when rows is None) -> normed rows."""
        self._f32(x, "residual stream")
        hidden = x.shape[-1]
        if delta is not None:
            self._act(delta, "residual addend")
            if delta.shape != x.shape:
                raise ValueError(f"residual addend {tuple(delta.shape)} does not match the stream {tuple(x.shape)}")
        if weight.dtype not in (torch.float32, self.dtype) or weight.numel() != hidden or weight.device.type != self.device.type:
            raise ValueError("norm weight: needs [hidden] in float32 or the compute dtype")
        n_rows = x.shape[0] if rows is None else rows.numel()
        if rows is not None:
            self._i32(rows, "norm rows")
        y = self.empty(n_rows, hidden)
        check(self.lib.cpm_add_rmsnorm(_ptr(x), _ptr(delta), float(alpha), _ptr(weight),
                                       1 if weight.dtype == torch.float32 else 0, _ptr(y), _ptr(rows), n_rows,
                                       hidden, float(eps), 1 if rows is None else 0, self.code, self._stream()),
              f"rmsnorm (hidden {hidden})")
        return y

    def residual_add(self, x: torch.Tensor, delta: torch.Tensor, alpha: float) -> None:
        self._f32(x, "residual stream")
        self._act(delta, "residual addend")
        if delta.shape != x.shape:
            raise ValueError("residual addend does not match the stream")
        check(self.lib.cpm_residual_add(_ptr(x), _ptr(delta), float(alpha), x.numel(), self.code, self._stream()),
              "residual add")

    def silu_mul(self, gu: torch.Tensor, interleave: int = 0) -> torch.Tensor:
        """gu [tokens, 2*inter] -> silu(gate) * up, [tokens, inter].  interleave 0: rows are
        [gate | up]; 8: blocks of 8 gate values followed by the 8 up values of the same features."""
        self._act(gu, "gate_up")
        n, two_i = gu.shape
        h = self.empty(n, two_i // 2)
        check(self.lib.cpm_silu_mul(_ptr(gu), _ptr(h), n, two_i // 2, interleave, self.code, self._stream()), "silu_mul")
        return h

    # ---- matrix products ----
    SKINNY_MAX_ROWS = int(os.environ.get("CPMCU_SKINNY_MAX_ROWS", "8"))   # most rows the weight-streaming product takes
    # From this many rows on the gated product runs on the tcgen05 kernel.  Its 128-row tiles are mostly empty for a
    # decode batch, but the product is bound by streaming the weights, not by the tensor cores: at 16 to 128 rows
    # it takes 51 us on the 8B gate_up shape (5.2 TB/s) with the activation applied in the epilogue, where the library
    # product takes 51 us and the activation kernel 4 us more.
    SKINNY_WIDE_BYTES = int(os.environ.get("CPMCU_SKINNY_WIDE_MB", "128")) << 20   # see _skinny_ok
    TCGEN05_MIN_ROWS = int(os.environ.get("CPMCU_TCGEN05_MIN_ROWS", "9"))
    MAX_DECODE_SPLITS = int(os.environ.get("CPMCU_MAX_SPLITS", "16"))     # most shares a sequence's pages are cut into
    LISTED_TILE_MIN_TOKENS = int(os.environ.get("CPMCU_LISTED_TILE_MIN", "32"))   # from here on prompt tokens share their blocks in tiles of eight
    SELECT_SCRATCH_BYTES = 64 << 20     # most scratch the sliced block selection may take (raw scores of all pooled keys)

    def _skinny_ok(self, M: int, K: int, N: int = 0) -> bool:
        """The weight-streaming product takes it: up to SKINNY_MAX_ROWS rows always; 9 to 16 rows (two tiles of token
        columns) while what its blocks read of the activations (every block all of them) stays small: at 16 rows
        the QKV, O and down products of the 8B sizes (not gate_up and the head), where it took 3.8 % off the step
        against the library's kernels (which stand outside the chain of dependent launches).  With four and eight tiles (up to 64 rows) the kernel
        lost to the library at every size tried, the 0.5B sizes included, and is not built."""
        if self.code != BF16 or K % 32 != 0:
            return False
        if M <= self.SKINNY_MAX_ROWS:
            return True
        return 0 < N and M <= 16 and -(-N // 16) * M * K * 2 <= self.SKINNY_WIDE_BYTES

    def linear(self, a: torch.Tensor, w: torch.Tensor, alpha: float = 1.0,
               out_f32: bool = False, result: bool = False) -> torch.Tensor:
        """alpha * a[M,K] @ w[N,K]^T -> [M,N] in the compute dtype, or fp32 when out_f32.  ``result``: the
        product is handed to the step's caller (see ``result``)."""
        self._act(a, "linear input")
        self._act(w, "linear weight")
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise ValueError(f"linear: input [*, {K}] against weight {tuple(w.shape)}")
        make = self.result if result else self.empty
        if self.code == F32:
            c = make(M, N, dtype=torch.float32)
            check(self.lib.cpm_gemm_f32(_ptr(a), _ptr(w), _ptr(c), M, N, K, K, K, N, float(alpha), self._stream()),
                  "fp32 matrix product")
            return c
        if self._skinny_ok(M, K, N):
            c = make(M, N, dtype=torch.float32 if out_f32 else self.dtype)
            check(self.lib.cpm_gemm_skinny_bf16(_ptr(w), _ptr(a), _ptr(c), M, N, K, float(alpha), 1 if out_f32 else 0,
                                                self._stream()), "skinny matrix product")
            return c
        c = make(M, N, dtype=torch.float32 if out_f32 else self.dtype)
        self._library_mm(a, w, c)
        if alpha != 1.0:
            c.mul_(alpha)
        return c

    def _library_mm(self, a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> None:
        """c = a @ w^T by the library (cuBLAS through torch), into a tensor of this library's own."""
        if c.dtype == a.dtype:
            torch.mm(a, w.t(), out=c)
        else:
            torch.mm(a, w.t(), out_dtype=c.dtype, out=c)

    def linear_tcgen05(self, a: torch.Tensor, w: torch.Tensor, gated: bool = False, pair: bool = False) -> torch.Tensor:
        """a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA operands, TMEM accumulator); with ``gated`` the
        weight is a gate_up matrix interleaved in blocks of 8 and the result is silu(gate) * up, [M, N/2].
        ``pair``: two blocks work on one 256 x 256 tile (cta_group::2)."""
        self._act(a, "linear input")
        self._act(w, "linear weight")
        M, K = a.shape
        N = w.shape[0]
        out = self.empty(M, N // 2 if gated else N)
        entry = self.lib.cpm_gemm_bf16_tcgen05_pair if pair else self.lib.cpm_gemm_bf16_tcgen05
        check(entry(_ptr(a), _ptr(w), _ptr(out), M, N, K, 2 if gated else 0, self.sm_count, self._stream()),
              f"tcgen05 matrix product [{M}x{K}] x [{N}x{K}]^T")
        return out

    def tcgen05_error(self) -> int:
        """Error code the tcgen05 product kernel recorded since the last call (0 = none); synchronises."""
        return int(self.lib.cpm_gemm_tcgen05_error())

    def gated_linear(self, a: torch.Tensor, w_gate_up: torch.Tensor, interleave: int) -> torch.Tensor:
        """silu(a @ gate^T) * (a @ up^T) for a gate_up matrix [2*inter, K] laid out as ``interleave`` says."""
        M, K = a.shape
        if interleave == 8 and self._skinny_ok(M, K, w_gate_up.shape[0]) and w_gate_up.shape[0] % 16 == 0:
            self._act(a, "linear input")
            self._act(w_gate_up, "gate_up weight")
            h = self.empty(M, w_gate_up.shape[0] // 2)
            check(self.lib.cpm_gemm_skinny_bf16(_ptr(w_gate_up), _ptr(a), _ptr(h), M, w_gate_up.shape[0], K, 1.0, 2,
                                                self._stream()), "gated skinny matrix product")
            return h
        few_tiles = M < 256 and w_gate_up.shape[0] // 256 < self.sm_count // 2     # a decode batch on a narrow model: too few blocks
        if (self.code == BF16 and interleave == 8 and self.use_tcgen05 and M >= self.TCGEN05_MIN_ROWS and K % 64 == 0
                and w_gate_up.shape[0] % 32 == 0 and a.data_ptr() % 16 == 0 and not few_tiles):
            # many rows (prefill): the tcgen05 product applies the activation in its epilogue
            return self.linear_tcgen05(a, w_gate_up, gated=True, pair=self.tcgen05_pair)
        return self.silu_mul(self.linear(a, w_gate_up), interleave)

    # ---- attention ----
    def rope_store(self, qkv: torch.Tensor, n_heads: int, n_kv: int, d: int, positions: torch.Tensor,
                   token_seq: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   inv_freq: Optional[torch.Tensor], magnitude: float, rot_dim: int) -> torch.Tensor:
        """Rotates q and k of qkv [tokens, (heads+2*kv)*d], stores k and v into the cache pages of
        each token's sequence, and returns the rotated q [tokens, heads, d]."""
        self._act(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (n_heads + 2 * n_kv) * d:
            raise ValueError("qkv row size does not match the head counts")
        if inv_freq is not None:
            self._f32(inv_freq, "inv_freq")
            if inv_freq.numel() != rot_dim // 2:
                raise ValueError("inv_freq needs rot_dim/2 entries")
        if k_cache is not None:
            self._act(k_cache, "key cache")
            self._act(v_cache, "value cache")
        q = self.empty(n, n_heads, d)
        check(self.lib.cpm_rope_store(_ptr(qkv), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(positions),
                                      _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                      _ptr(inv_freq), float(magnitude), n, n_heads, n_kv, d, rot_dim, self.code,
                                      self._stream()), "rope_store")
        return q

    def attention_generic(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          positions: torch.Tensor, token_seq: torch.Tensor, slots: torch.Tensor,
                          page_table: torch.Tensor, n_kv: int, scale: float, window: int = 0,
                          block_list: Optional[torch.Tensor] = None, block_size: int = 0) -> torch.Tensor:
        """q [tokens, heads, d] against the cached keys of each token's sequence -> [tokens, heads*d]."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        out = self.empty(n, n_heads * d)
        list_cap = 0
        if block_list is not None:
            self._i32(block_list, "block list")
            list_cap = block_list.shape[-1]
        check(self.lib.cpm_attention_generic(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(positions),
                                             _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                             _ptr(block_list), list_cap, block_size, window, n, n_heads, n_kv, d,
                                             float(scale), self.code, self._stream()),
              f"attention (head_dim {d}, {n_heads} heads, {n_kv} kv heads)")
        return out

    # ---- sampling ----
    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               top_p: Optional[torch.Tensor] = None, seed: int = 0, seq_key: Optional[torch.Tensor] = None,
               step_key: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits [rows, vocab] -> int32 [rows]; greedy where temperature is absent or 0."""
        self._f32(logits, "logits")
        rows, vocab = logits.shape
        if out is None:
            out = self.result(rows, dtype=torch.int32)
        check(self.lib.cpm_sample_rows(_ptr(logits), logits.stride(0), rows, vocab, _ptr(out), _ptr(temperature),
                                       _ptr(top_p), ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), _ptr(seq_key),
                                       _ptr(step_key), self._stream()), "sample")
        return out

    def attention(self, ctx, q: torch.Tensor, lane, n_kv: int, scale: float, window: int = 0,
                  block_list: Optional[torch.Tensor] = None, block_size: int = 0) -> torch.Tensor:
        """Attention of the step's queries over their sequences' cached keys; picks the kernel."""
        n, n_heads, d = q.shape
        if self.code == BF16 and block_list is None and not window and d in FAST_HEAD_DIMS:
            if ctx.is_decode:
                return self.decode_attention(q, lane.k, lane.v, ctx.kv_len_dev, ctx.slot_dev, lane.page_table,
                                             n_kv, scale)
            tiles = ctx.q_tiles
            if (tiles is not None and self.use_tcgen05_attention and (n_heads // n_kv) % 2 == 0
                    and (d == 128 or (d == 64 and ctx.max_kv_len >= 1024))):      # short prompts of head size 64: the smaller tiles win
                return self.prefill_attention_tcgen05(q, lane.k, lane.v, tiles, ctx.cu_q, ctx.kv_len_dev, ctx.slot_dev,
                                                      lane.page_table, n_kv, scale,
                                                      self.prefill_key_shares(ctx.q_lens, ctx.max_kv_len, n_heads))
            if tiles is not None:
                return self.prefill_attention(q, lane.k, lane.v, tiles, ctx.cu_q, ctx.kv_len_dev, ctx.slot_dev,
                                              lane.page_table, n_kv, scale)
        if (self.code == BF16 and block_list is not None and block_size == PAGE_TOKENS and not window
                and d in FAST_HEAD_DIMS):
            return self.listed_attention(q, lane.k, lane.v, ctx.positions, ctx.token_seq, ctx.slot_dev,
                                         lane.page_table, block_list, n_kv, scale,
                                         tiles=not ctx.is_decode and n >= self.LISTED_TILE_MIN_TOKENS)
        return self.attention_generic(q, lane.k, lane.v, ctx.positions, ctx.token_seq, ctx.slot_dev,
                                      lane.page_table, n_kv, scale, window, block_list, block_size)

    # ---- block-sparse selection ----
    def pool_keys(self, ctx, lane, n_kv: int, d: int, kernel: int, stride: int) -> None:
        """Stores the mean-pooled keys whose windows this step's tokens complete."""
        check(self.lib.cpm_pool_keys(_ptr(lane.k), _ptr(lane.pooled), _ptr(ctx.positions), _ptr(ctx.token_seq),
                                     _ptr(ctx.slot_dev), _ptr(lane.page_table), lane.page_table.shape[1],
                                     ctx.n_tokens, n_kv, d, kernel, stride, self.code, self._stream()), "pool_keys")

    def select_blocks(self, ctx, q: torch.Tensor, lane, n_kv: int, scale: float, sparse) -> Tuple[torch.Tensor, int]:
        """(block list int32 [tokens, kv_heads, cap], block size) for the step's queries."""
        n, n_heads, d = q.shape
        bs, stride = sparse["block_size"], sparse["kernel_stride"]
        local_blocks = sparse["window_size"] // bs
        cap = sparse["topk"] + local_blocks + 2
        # an upper bound on the pooled keys a query sees; it sizes the sort of the candidate blocks (8 bytes of shared
        # memory per block), not the walk over the pooled keys, which follows each query's own position
        longest = ctx.max_kv_len          # in a recorded step an upper bound (the cache's capacity per sequence, or less)
        max_entries = max(1, longest // stride + 1)
        lists = self.empty(n, n_kv, cap, dtype=torch.int32)
        # few queries (a decode step): share every query's pooled keys out over many blocks, in two kernels
        scratch, n_slices = None, 0
        units = n * n_kv
        if (self.code == BF16 and units * 2 <= self.sm_count and n_heads // n_kv <= 16 and d in FAST_HEAD_DIMS
                and units * max_entries * 64 <= self.SELECT_SCRATCH_BYTES):
            n_slices = max(1, min(2 * self.sm_count // units, (max_entries + 63) // 64))
            scratch = self.empty(self.lib.cpm_select_blocks_scratch_floats(n, n_kv, max_entries, n_slices), dtype=torch.float32)
        check(self.lib.cpm_select_blocks(_ptr(q), _ptr(lane.pooled), _ptr(ctx.positions), _ptr(ctx.token_seq),
                                         _ptr(ctx.slot_dev), _ptr(lane.page_table), lane.page_table.shape[1],
                                         _ptr(lists), cap, n, n_heads, n_kv, d, float(scale), sparse["kernel_size"],
                                         stride, bs, sparse.get("init_blocks", 1), sparse["topk"], local_blocks,
                                         sparse.get("dense_len", 0), max_entries, self.code, _ptr(scratch), n_slices,
                                         self._stream()),
              f"select_blocks ({max_entries} pooled keys)")
        if scratch is not None:
            LAUNCHES_EXTRA[0] += 1
        return lists, bs

    def advance_decode(self, ids, positions, kv_len, step_key, sampled, live) -> None:
        check(self.lib.cpm_advance_decode(_ptr(ids), _ptr(positions), _ptr(kv_len), _ptr(step_key), _ptr(sampled),
                                          _ptr(live), ids.numel(), self._stream()), "advance_decode")

    # ---- bf16 tensor-core attention ----
    def decode_splits(self, n_seqs: int, n_heads: int, n_kv: int) -> int:
        """How many shares a sequence's pages are cut into: the decode attention kernel holds one
        block per SM (its page buffers fill the shared memory), so aim at one wave of blocks."""
        m_tiles = (n_heads // n_kv + 15) // 16
        units = max(1, n_seqs * n_kv * m_tiles)
        return max(1, min(self.MAX_DECODE_SPLITS, self.sm_count // units))

    def decode_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor,
                         slots: torch.Tensor, page_table: torch.Tensor, n_kv: int, scale: float,
                         n_splits: Optional[int] = None) -> torch.Tensor:
        """One query token per sequence: q [seqs, heads, d] -> [seqs, heads*d]."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        if n_splits is None:
            n_splits = self.decode_splits(n, n_heads, n_kv)
        floats = self.lib.cpm_decode_attention_scratch_floats(n, n_heads, n_kv, d, n_splits)
        scratch = self.empty(floats, dtype=torch.float32)
        out = self.empty(n, n_heads * d)
        check(self.lib.cpm_decode_attention_bf16(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(kv_len),
                                                 _ptr(slots), _ptr(page_table), page_table.shape[1], _ptr(scratch),
                                                 n, n_heads, n_kv, d, n_splits, float(scale), self._stream()),
              f"decode attention (head_dim {d})")
        if n_splits > 1:
            LAUNCHES_EXTRA[0] += 1       # the launcher starts two kernels: the shares, then their combination
        return out

    FUSED_ROPE_HEAD_DIMS = (64, 128)      # head sizes whose rotary pairs lie in one thread's fragments of the decode kernel

    def fused_decode_ok(self, ctx, d: int, rot_dim: int, window: int, sparse) -> bool:
        """Whether a decode step's rotation and cache store are done by the attention kernel itself.  It saves a
        launch, which counts where launches are what a step waits for (steps that are not recorded into a graph).
        Inside a graph the separate rotary kernel overlaps with its neighbours and the fused kernel is 0.7 % slower
        on the 8B decode step (3.537 against 3.501 ms at batch 8), so recorded steps keep the two kernels.
        CPMCU_FUSED_ROPE=1 / 0 forces the choice."""
        forced = os.environ.get("CPMCU_FUSED_ROPE")
        want = (forced != "0") if forced is not None else not ctx.captured
        return (want and self.code == BF16 and ctx.is_decode and not window and sparse is None
                and d in self.FUSED_ROPE_HEAD_DIMS and rot_dim in (0, d))

    def decode_attention_rope(self, qkv: torch.Tensor, lane, kv_len: torch.Tensor, slots: torch.Tensor, n_heads: int,
                              n_kv: int, d: int, scale: float, inv_freq: Optional[torch.Tensor], magnitude: float,
                              write_cache: bool, n_splits: Optional[int] = None) -> torch.Tensor:
        """A decode step's attention straight from the fused product qkv [seqs, (heads + 2 kv) * d]: the kernel
        rotates q and the new key (position = keys - 1), stores the new key and value into the sequence's page (when
        ``write_cache``) and attends.  One launch less than rope_store followed by decode_attention."""
        self._act(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (n_heads + 2 * n_kv) * d:
            raise ValueError("qkv row size does not match the head counts")
        if inv_freq is not None:
            self._f32(inv_freq, "inv_freq")
            if inv_freq.numel() != d // 2:
                raise ValueError("inv_freq needs head_dim/2 entries")
        if n_splits is None:
            n_splits = self.decode_splits(n, n_heads, n_kv)
        floats = self.lib.cpm_decode_attention_scratch_floats(n, n_heads, n_kv, d, n_splits)
        scratch = self.empty(floats, dtype=torch.float32)
        out = self.empty(n, n_heads * d)
        check(self.lib.cpm_decode_attention_rope_bf16(_ptr(qkv), _ptr(lane.k), _ptr(lane.v), _ptr(out), _ptr(kv_len),
                                                      _ptr(slots), _ptr(lane.page_table), lane.page_table.shape[1],
                                                      _ptr(scratch), n, n_heads, n_kv, d, n_splits, float(scale),
                                                      _ptr(inv_freq), float(magnitude), 1 if write_cache else 0,
                                                      self._stream()), f"decode attention with rotation (head_dim {d})")
        if n_splits > 1:
            LAUNCHES_EXTRA[0] += 1
        return out

    def prefill_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tiles,
                          cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                          n_kv: int, scale: float) -> torch.Tensor:
        """q [tokens, heads, d] packed by sequence -> [tokens, heads*d]; tiles = (tile_seq, tile_row, count)
        lists the query tiles of PREFILL_TILE_ROWS tokens."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        tile_seq, tile_row, n_tiles = tiles
        out = self.empty(n, n_heads * d)
        check(self.lib.cpm_prefill_attention_bf16(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq),
                                                  _ptr(tile_row), n_tiles, _ptr(cu_q), _ptr(kv_len), _ptr(slots),
                                                  _ptr(page_table), page_table.shape[1], n_heads, n_kv, d,
                                                  float(scale), self._stream()), f"prefill attention (head_dim {d})")
        return out


    def prefill_attention_tcgen05(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tiles,
                                  cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor,
                                  page_table: torch.Tensor, n_kv: int, scale: float, n_splits: int = 1) -> torch.Tensor:
        """The same as ``prefill_attention`` on the tcgen05 tensor cores: head size 128 or 64 and an even number
        of query heads per key/value head.  ``n_splits`` > 1 shares the keys of every tile out over that many
        blocks (a short chunk after a long history would otherwise keep few SMs busy for long)."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        tile_seq, tile_row, n_tiles = tiles
        out = self.empty(n, n_heads * d)
        scratch = self.empty(n_splits * n * n_heads * (d + 2), dtype=torch.float32) if n_splits > 1 else None
        check(self.lib.cpm_prefill_attention_tcgen05(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq),
                                                     _ptr(tile_row), n_tiles, _ptr(cu_q), _ptr(kv_len), _ptr(slots),
                                                     _ptr(page_table), page_table.shape[1], n, k_cache.shape[0],
                                                     n_heads, n_kv, d, float(scale), _ptr(scratch), n_splits, self._stream()),
              f"tcgen05 prefill attention (head_dim {d})")
        return out

    def prefill_key_shares(self, q_lens, max_kv_len: int, n_heads: int) -> int:
        """How many blocks share the keys of a query tile in the tcgen05 attention: one, unless the step's 128-token
        tiles times head pairs leave most SMs idle and there are enough keys (at least 8 steps of 128 per share)."""
        blocks = sum((int(n) + 127) // 128 for n in q_lens) * max(1, n_heads // 2)
        steps = (int(max_kv_len) + 127) // 128
        if blocks * 2 > self.sm_count or steps < 16:
            return 1
        return max(1, min(self.sm_count // blocks, steps // 8, 16))

    def attention_tcgen05_error(self) -> int:
        """Error code the tcgen05 attention kernel recorded since the last call (0 = none); synchronises."""
        return int(self.lib.cpm_attention_tcgen05_error())

    def raise_on_kernel_error(self) -> None:
        """The tcgen05 kernels bound every wait and record a code instead of hanging; this turns a recorded
        code into an exception.  It synchronises the device: call it where the host waits anyway."""
        gemm, attn = self.tcgen05_error(), self.attention_tcgen05_error()
        if gemm or attn:
            raise RuntimeError(f"a tcgen05 kernel gave up waiting on a barrier (product: code {gemm}, attention: code "
                               f"{attn}); the results of this step are not valid")
        self.raise_on_bounds_error()
        arena = self.workspace.persistent.arena if self.workspace is not None else None
        if arena is not None and arena.guards:
            arena.check_guards()
        if int(self.lib.cpm_listed_tile_error()):
            raise RuntimeError("the block-list attention of a prompt chunk gave up waiting on a barrier; the results of "
                               "this step are not valid")
        if int(self.lib.cpm_select_blocks_error()):
            raise RuntimeError("block selection met a query with more candidate key blocks than the launch made room "
                               "for (a sequence longer than the bound the step gave); the results of this step are not valid")

    # ---- the checked build (CPMCU_CHECK_BOUNDS=1) ----
    def set_page_limit(self, n_pages: int) -> None:
        """Tells the checked kernels how many pages the cache in use holds (no-op in the ordinary build)."""
        if (getattr(self.lib, "checked_files", None) and n_pages != getattr(self, "_page_limit", None)
                and not torch.cuda.is_current_stream_capturing()):
            for _, _, limit in self.lib.checked_files:
                limit(int(n_pages))
            self._page_limit = n_pages

    def raise_on_bounds_error(self) -> None:
        """The checked build's records: a page index or page number out of range that a kernel met (and did not
        follow).  Synchronises."""
        for name, error, _ in getattr(self.lib, "checked_files", None) or ():
            rec = (ctypes.c_int * 4)()
            if error(ctypes.byref(rec)):
                what = "a page-table index beyond the table" if rec[0] == 1 else "a page number beyond the cache"
                raise RuntimeError(f"checked build: a kernel of {name}.cu met {what}: index {rec[1]}, value {rec[2]}, "
                                   f"limit {rec[3]}; it used page 0 instead, the step's results are not valid")

    def listed_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                         token_seq: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                         block_list: torch.Tensor, n_kv: int, scale: float, tiles: bool = False) -> torch.Tensor:
        """Attention of every token over the 64-token key blocks its list names (block-sparse).  ``tiles``: the
        tokens are those of prompts (consecutive tokens mostly of one sequence); eight of them then share the
        blocks they bring from the cache."""
        self._act(q, "q")
        self._i32(block_list, "block list")
        n, n_heads, d = q.shape
        out = self.empty(n, n_heads * d)
        if (tiles and self.use_tcgen05_attention and self.use_tcgen05_listed and d == 128 and n_heads == 16 * n_kv
                and page_table.shape[1] <= self.lib.cpm_listed_attention_tcgen05_max_pages()):
            # prompt tokens of the long-context shape: eight tokens x sixteen heads are one tensor-core tile
            check(self.lib.cpm_listed_attention_tcgen05(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(positions),
                                                        _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                                        k_cache.shape[0], _ptr(block_list), block_list.shape[-1], n, n_heads,
                                                        n_kv, d, float(scale), self._stream()),
                  "block-list attention on tcgen05")
            return out
        n_splits = 1 if tiles else self.decode_splits(n, n_heads, n_kv)      # few tokens (decode): share a token's blocks out
        scratch = None
        if n_splits > 1:
            scratch = self.empty(self.lib.cpm_decode_attention_scratch_floats(n, n_heads, n_kv, d, n_splits),
                                 dtype=torch.float32)
        check(self.lib.cpm_listed_attention_bf16(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(positions),
                                                 _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                                 _ptr(block_list), block_list.shape[-1], n, n_heads, n_kv, d,
                                                 float(scale), _ptr(scratch), n_splits, 1 if tiles else 0, self._stream()),
              f"block-list attention (head_dim {d})")
        return out


LAUNCHES_EXTRA = library.LAUNCHES
