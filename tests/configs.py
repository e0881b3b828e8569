"""The tiny configurations the tests use, as raw config.json dictionaries.

Tiny A and tiny B differ in every size and option: layers, hidden size, head counts and
group size, head_dim, intermediate size (no multiple of 128), vocabulary, plain rotary
against LongRoPE, eps, the three scales, tied against untied head, dense against sparse
attention.
"""
import math


def tiny_a() -> dict:
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 16, "intermediate_size": 176, "vocab_size": 512,
        "rope_theta": 10000.0, "max_position_embeddings": 128, "rms_norm_eps": 1e-6,
        "scale_emb": 12, "dim_model_base": 16, "scale_depth": 1.4, "tie_word_embeddings": True,
        "hidden_act": "silu", "torch_dtype": "float32", "eos_token_id": 2,
    }


def long_factors(n: int, lo: float, hi: float) -> list:
    # ascending, not evenly spaced
    return [lo + (hi - lo) * ((i / (n - 1)) ** 1.5) for i in range(n)]


def tiny_b(sparse: bool = True) -> dict:
    cfg = {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 1,
        "head_dim": 32, "intermediate_size": 320, "vocab_size": 1000,
        "rope_theta": 1000000.0, "max_position_embeddings": 256, "rms_norm_eps": 1e-5,
        "rope_scaling": {"rope_type": "longrope", "short_factor": [1.0] * 16,
                         "long_factor": long_factors(16, 1.0, 8.0), "original_max_position_embeddings": 64},
        "scale_emb": 8, "dim_model_base": 32, "scale_depth": 1.0, "tie_word_embeddings": False,
        "hidden_act": "silu", "torch_dtype": "bfloat16", "eos_token_id": [1, 7],
    }
    if sparse:
        cfg["sparse_config"] = {"kernel_size": 8, "kernel_stride": 4, "block_size": 16, "init_blocks": 1,
                                "topk": 2, "window_size": 32, "dense_len": 64}
    return cfg


def tiny_c() -> dict:
    """Odd sizes: hidden and vocabulary that are no power of two, three query heads per
    key-value head, head_dim 48, no scale keys at all."""
    return {
        "architectures": ["MiniCPMForCausalLM"],
        "num_hidden_layers": 2, "hidden_size": 72, "num_attention_heads": 6, "num_key_value_heads": 2,
        "head_dim": 48, "intermediate_size": 100, "vocab_size": 777,
        "max_position_embeddings": 512, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    }


def tiny_d() -> dict:
    """Sparse attention with blocks of a whole cache page (64 tokens), as the 8B configuration has:
    the block-list kernel of the bf16 path takes these."""
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 2, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 2,
        "head_dim": 32, "intermediate_size": 160, "vocab_size": 640,
        "rope_theta": 10000.0, "max_position_embeddings": 1024, "rms_norm_eps": 1e-6,
        "scale_emb": 4, "dim_model_base": 48, "scale_depth": 1.2, "tie_word_embeddings": True,
        "sparse_config": {"kernel_size": 32, "kernel_stride": 16, "block_size": 64, "init_blocks": 1, "topk": 3,
                          "window_size": 64, "dense_len": 100},
    }


def tiny_e() -> dict:
    """Head size 128 with two query heads per key-value head and sizes in multiples of 64: the shapes that
    the tcgen05 attention and the tcgen05 gated product of the bf16 path take (from 256 prompt tokens on)."""
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 128, "intermediate_size": 160, "vocab_size": 900,
        "rope_theta": 50000.0, "max_position_embeddings": 2048, "rms_norm_eps": 2e-6,
        "scale_emb": 6, "dim_model_base": 96, "scale_depth": 1.1, "tie_word_embeddings": False,
    }


def tiny_f() -> dict:
    """Head size 64 with four query heads per key-value head: the tcgen05 attention's other head size, which the
    engine takes from 1,024 keys on."""
    return {
        "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
        "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 8, "num_key_value_heads": 2,
        "head_dim": 64, "intermediate_size": 96, "vocab_size": 500,
        "rope_theta": 10000.0, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5,
        "scale_emb": 3, "dim_model_base": 64, "scale_depth": 1.3, "tie_word_embeddings": True,
    }
