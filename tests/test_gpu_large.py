"""Models of the real layer sizes (MiniCPM4-0.5B whole, MiniCPM4-8B with two layers) with random
weights made on the device: the bfloat16 path against the engine's own float32 path, which the other
tests tie to the plain implementation.  (A plain CPU run at these sizes takes minutes per sequence.)
Shapes that only occur here: head_dim 64 and 128, 8 and 16 query heads per key-value head, a
vocabulary of 73,448 that is no multiple of 16, intermediate sizes 4,096 and 16,384."""
import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm", "vocab_size": 73448, "rope_theta": 10000.0,
        "max_position_embeddings": 65536, "rms_norm_eps": 1e-6, "scale_emb": 12, "dim_model_base": 256, "scale_depth": 1.4,
        "hidden_act": "silu"}
HALF_B = dict(BASE, num_hidden_layers=24, hidden_size=1024, num_attention_heads=16, num_key_value_heads=2, head_dim=64,
              intermediate_size=4096, tie_word_embeddings=True)
EIGHT_B = dict(BASE, num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=2, head_dim=128,
               intermediate_size=16384, tie_word_embeddings=False)


def _long_factors(n):
    g = torch.Generator().manual_seed(3)
    return sorted((1.0 + 39.0 * torch.rand(n, generator=g)).tolist())


def _engine(cfgd, dtype, seed):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    half = cfgd["head_dim"] // 2
    cfgd = dict(cfgd, rope_scaling={"rope_type": "longrope", "long_factor": _long_factors(half), "short_factor": [1.0] * half,
                                    "original_max_position_embeddings": 32768})
    arch = architecture("MiniCPMForCausalLM")
    cfg = arch.config_class.from_dict(cfgd)
    model = build_model(arch, cfg, dtype, "cuda:0")
    # the same bf16-rounded values for both paths: drawn in bf16, widened for the float32 model
    w = random_tensors(model.weight_specs(), seed, torch.bfloat16, std=0.02, device="cuda:0")
    model.load_weights({k: v.to(dtype) for k, v in w.items()})
    del w
    cache = Cache(model.cache_needs(), max_tokens=64 * 16, dtype=dtype, device="cuda:0")
    return cfg, Stepper(model, cache, chunk_tokens=256)


def _run(cfgd, dtype, seqs, tail):
    from cpmcu_b200.engine import SequenceStep

    cfg, st = _engine(cfgd, dtype, 4)
    slots = st.open(len(seqs))
    rows = [[] for _ in seqs]
    out = st.step([SequenceStep(s, ids[:-tail], [0, len(ids) - tail - 1]) for s, ids in zip(slots, seqs)])
    for i in range(len(seqs)):
        rows[i].append(out[2 * i:2 * i + 2])
    for t in range(tail):
        out = st.step([SequenceStep(s, [ids[len(ids) - tail + t]], [0]) for s, ids in zip(slots, seqs)])
        for i in range(len(seqs)):
            rows[i].append(out[i:i + 1])
    result = [torch.cat(r).cpu() for r in rows]
    del st
    torch.cuda.empty_cache()
    return result


@pytest.mark.parametrize("name,cfgd", [("0.5B", HALF_B), ("8B-2-layers", EIGHT_B)])
def test_real_layer_sizes_bf16_against_float32(name, cfgd):
    seqs = [helpers.random_ids(cfgd["vocab_size"], n, n) for n in (300, 70, 129)]
    want = _run(cfgd, torch.float32, seqs, tail=6)
    got = _run(cfgd, torch.bfloat16, seqs, tail=6)
    for i, (g, w) in enumerate(zip(got, want)):
        assert torch.isfinite(g).all()
        # Root-mean-square error against the root-mean-square logit: the rounding noise of the bf16
        # pipeline itself (about ten roundings per layer of 2^-9 each).
        rms = float((g - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt())
        assert rms < 2.5e-2, (name, i, rms)
        # The largest error against the largest logit.  Over 8 rows of 73,448 logits the largest of
        # ~600,000 noise samples is compared with the largest of as many logits, so this ratio sits
        # near the rms ratio (measured 1.1e-2 to 1.4e-2 at the 8B sizes, 2e-3 at the 0.5B sizes); the
        # bound is the bf16 bound of the small models with room for that tail.
        err = helpers.rel_err(g, w)
        assert err < 2 * helpers.TOL["bfloat16"], (name, i, err)
