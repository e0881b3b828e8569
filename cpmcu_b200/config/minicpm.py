"""Typed configuration of the MiniCPM4 architecture (``MiniCPMForCausalLM``).

Every size and constant the model uses is a field here, read from the keys the
architecture's own ``config.json`` uses.  The reference derives the three muP
scales in cpmcu/llm.py:67-69 and takes the InfLLM-v2 knobs from command-line flags
(cpmcu/common/args.py:73-83); here the sparse knobs are the ``sparse_config``
object of config.json.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, FieldReader, read_config_json


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json; only the ``longrope`` rule exists for this architecture."""

    rope_type: str
    long_factor: List[float]
    short_factor: List[float]
    original_max_position_embeddings: int

    def to_json(self) -> Dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "long_factor": list(self.long_factor),
            "short_factor": list(self.short_factor),
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class SparseConfig:
    """``sparse_config`` of config.json: InfLLM-v2 block-sparse attention.

    kernel_size/kernel_stride: window and step of the mean-pooled ("compressed") keys
    (32/16 in src/model/minicpm4/minicpm4_kvcache.cuh:6-30); block_size: tokens per
    selectable block (64, minicpm4_kvcache.cuh:163-168); init_blocks: leading blocks
    always attended (``sink_window_size``); topk: blocks selected per query and
    key-value head, the leading blocks included; window_size: tokens of the local
    window that is always attended; dense_len: queries whose key count does not
    exceed it use dense attention (``sparse_switch``).
    """

    kernel_size: int
    kernel_stride: int
    block_size: int
    init_blocks: int
    topk: int
    window_size: int
    dense_len: int

    def to_json(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclass(frozen=True)
class MiniCPMConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    hidden_act: str
    scale_emb: float
    dim_model_base: float
    scale_depth: Optional[float]
    tie_word_embeddings: bool
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Optional[RopeScaling]
    sparse_config: Optional[SparseConfig]
    torch_dtype: str
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None

    architecture = "MiniCPMForCausalLM"

    # ---- derived constants (cpmcu/llm.py:67-69) ----
    @property
    def residual_scale(self) -> float:
        if self.scale_depth is None:
            return 1.0
        return self.scale_depth / math.sqrt(self.num_hidden_layers)

    @property
    def logit_scale(self) -> float:
        return self.dim_model_base / self.hidden_size

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ---- reading ----
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "MiniCPMConfig":
        r = FieldReader(data)
        vocab = r.integer("vocab_size", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        layers = r.integer("num_hidden_layers", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        inter = r.integer("intermediate_size", minimum=1)
        eps = r.number("rms_norm_eps", positive=True)
        head_dim = r.integer("head_dim", default=None, minimum=1)
        act = r.string("hidden_act", default="silu", choices=("silu",))
        scale_emb = r.number("scale_emb", default=1.0)
        dim_model_base = r.number("dim_model_base", default=None, positive=True)
        scale_depth = r.number("scale_depth", default=None, positive=True)
        tie = r.boolean("tie_word_embeddings", default=False)
        theta = r.number("rope_theta", default=10000.0, positive=True)
        max_pos = r.integer("max_position_embeddings", minimum=1)
        dtype = r.string("torch_dtype", default="bfloat16")
        eos = r.int_or_ints("eos_token_id", default=[])
        bos = r.integer("bos_token_id", default=None)

        if head_dim is None and hidden is not None and heads is not None:
            r.check(hidden % heads == 0,
                    f"'hidden_size' ({hidden}) is not a multiple of 'num_attention_heads' ({heads}) and no 'head_dim' is given")
            head_dim = hidden // heads
        if dim_model_base is None and hidden is not None:
            dim_model_base = float(hidden)
        if heads is not None and kv_heads is not None:
            r.check(heads % kv_heads == 0,
                    f"'num_attention_heads' ({heads}) is not a multiple of 'num_key_value_heads' ({kv_heads})")
        if head_dim is not None:
            r.check(head_dim % 2 == 0, f"'head_dim' ({head_dim}) must be even for rotary pairs")

        rope = None
        rs = r.child("rope_scaling")
        if rs is not None:
            kind = rs.string("rope_type", default=None)
            if kind is None:
                kind = rs.string("type", default=None)
            rs.used.update({"rope_type", "type", "factor"})
            if kind is None:
                rs.problems.append(f"{rs.where}: needs 'rope_type' (or 'type')")
            elif kind != "longrope":
                rs.problems.append(f"{rs.where}: unknown rope_type {kind!r}; known: ['longrope']")
            long_f = rs.numbers("long_factor")
            short_f = rs.numbers("short_factor")
            orig = rs.integer("original_max_position_embeddings", default=None, minimum=2)
            if orig is None:
                orig = r.integer("original_max_position_embeddings", default=None, minimum=2)
            if orig is None:
                rs.problems.append(f"{rs.where}: needs 'original_max_position_embeddings'")
            if head_dim is not None:
                for name, f in (("long_factor", long_f), ("short_factor", short_f)):
                    if f is not None:
                        rs.check(len(f) == head_dim // 2,
                                 f"'{name}' has {len(f)} entries, head_dim/2 = {head_dim // 2} are needed")
                        rs.check(all(x > 0 for x in f), f"'{name}' entries must be > 0")
            r.absorb(rs)
            if not rs.problems:
                rope = RopeScaling(kind, long_f, short_f, orig)

        sparse = None
        sc = r.child("sparse_config")
        if sc is not None:
            ks = sc.integer("kernel_size", minimum=1)
            st = sc.integer("kernel_stride", minimum=1)
            bs = sc.integer("block_size", minimum=1)
            ib = sc.integer("init_blocks", default=1, minimum=0)
            tk = sc.integer("topk", minimum=1)
            ws = sc.integer("window_size", minimum=1)
            dl = sc.integer("dense_len", default=0, minimum=0)
            if not sc.problems:
                sc.check(ks % st == 0, f"'kernel_size' ({ks}) must be a multiple of 'kernel_stride' ({st})")
                sc.check(bs % st == 0, f"'block_size' ({bs}) must be a multiple of 'kernel_stride' ({st})")
                sc.check(ks <= bs, f"'kernel_size' ({ks}) must not exceed 'block_size' ({bs})")
                sc.check(ws % bs == 0 and ws >= bs,
                         f"'window_size' ({ws}) must be a positive multiple of 'block_size' ({bs})")
                sc.check(tk >= ib, f"'topk' ({tk}) counts the 'init_blocks' ({ib}) and must not be smaller")
            r.absorb(sc)
            if not sc.problems:
                sparse = SparseConfig(ks, st, bs, ib, tk, ws, dl)

        r.finish()
        return cls(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            intermediate_size=inter, rms_norm_eps=eps, hidden_act=act, scale_emb=scale_emb,
            dim_model_base=dim_model_base, scale_depth=scale_depth, tie_word_embeddings=tie,
            rope_theta=theta, max_position_embeddings=max_pos, rope_scaling=rope,
            sparse_config=sparse, torch_dtype=dtype, eos_token_ids=eos, bos_token_id=bos,
        )

    @classmethod
    def from_json(cls, model_dir_or_file: str) -> "MiniCPMConfig":
        return cls.from_dict(read_config_json(model_dir_or_file))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json of a model folder holding this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "minicpm",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rms_norm_eps": self.rms_norm_eps,
            "hidden_act": self.hidden_act,
            "scale_emb": self.scale_emb,
            "dim_model_base": self.dim_model_base,
            "tie_word_embeddings": self.tie_word_embeddings,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_scaling": self.rope_scaling.to_json() if self.rope_scaling else None,
            "sparse_config": self.sparse_config.to_json() if self.sparse_config else None,
            "torch_dtype": self.torch_dtype,
        }
        if self.scale_depth is not None:
            d["scale_depth"] = self.scale_depth
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d
