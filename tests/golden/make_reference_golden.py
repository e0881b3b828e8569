#!/usr/bin/env python3
"""Logits of the unmodified reference (OpenBMB/CPM.cu) on tiny random models, kept as golden files.

The reference has no CPU path: its model code is CUDA behind ``cpmcu.C``.  So the comparison of the
plain implementation (tests/plain) with the reference's own code is made once on a GPU, here, and its
small outputs are committed beside this script; tests/test_cpu_golden.py then checks the plain
implementation against them on the CPU at every run.  The reference is the build that
``bench.py --impl reference`` uses (installed under baseline/_ref); run on a machine with a GPU:

    PYTHONPATH=baseline/_ref python tests/golden/make_reference_golden.py --out tests/golden

What is run is the reference's stock path through its public class: ``cpmcu.llm.LLM`` with
``init_storage``, its loader (every tensor from a safetensors file by its Hugging Face name), ``prefill``
in chunks of 32 tokens and ``decode`` one token at a time, in bfloat16, without CUDA graphs.  The rotary
table is the one thing handed over: ``load_from_hf`` asks another package for it under a name
("default") that the installed version of that package no longer has, so the loader's two halves are
called here as ``load_from_hf`` calls them (cpmcu/llm.py:178-192), with inv_freq[c] = theta^(-2c/d)
for the table.  Nothing of cpmcu_b200 is imported.

The models (two, differing in every size the reference's kernels allow: its attention is built for
head sizes 64 and 128) are given to the reference as ``llama`` configurations that carry MiniCPM's
three scale keys, which is how it reads them (cpmcu/llm.py:62-69).  Plain rotary encoding only: with
LongRoPE the reference drops the attention factor (cpmcu/llm.py:190-192), which the plain
implementation and the engine apply, so that case is not a parity case.

A golden file holds: the configuration (JSON), the seed of the weights, the token ids, the positions
whose logits were taken, and the logits [positions, vocab] as float32 (the reference returns bfloat16).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

import numpy as np
import torch

CONFIGS = {
    "hd64": {
        "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
        "intermediate_size": 352, "vocab_size": 512, "rope_theta": 10000.0, "max_position_embeddings": 512,
        "rms_norm_eps": 1e-6, "scale_emb": 12, "dim_model_base": 32, "scale_depth": 1.4, "tie_word_embeddings": False,
    },
    "hd128": {
        "num_hidden_layers": 3, "hidden_size": 384, "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 128,
        "intermediate_size": 608, "vocab_size": 776, "rope_theta": 50000.0, "max_position_embeddings": 512,
        "rms_norm_eps": 1e-5, "scale_emb": 7, "dim_model_base": 64, "scale_depth": 2.2, "tie_word_embeddings": True,
    },
}
SEEDS = {"hd64": 11, "hd128": 12}
PROMPT, DECODED = 75, 12                  # the prompt is prefilled in chunks of 32; then tokens one by one
PREFIXES = (1, 9, 32, 33, 64, 75)         # prompts whose last position's logits are kept (chunk edges among them)


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors by Hugging Face name: matrices N(0, 0.05), norm weights 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(rows, cols):
        return (torch.randn(rows, cols, generator=g) * 0.05).to(torch.bfloat16)

    def vec(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)

    w = {"model.embed_tokens.weight": mat(V, H)}
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        w[p + "input_layernorm.weight"] = vec(H)
        w[p + "self_attn.q_proj.weight"] = mat(nh * d, H)
        w[p + "self_attn.k_proj.weight"] = mat(nkv * d, H)
        w[p + "self_attn.v_proj.weight"] = mat(nkv * d, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, nh * d)
        w[p + "post_attention_layernorm.weight"] = vec(H)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = vec(H)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, H)
    return w


def make_tokens(cfg: dict, seed: int) -> list:
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, cfg["vocab_size"], (PROMPT + DECODED,), generator=g).tolist()


def write_folder(folder: str, cfg: dict, weights: dict) -> None:
    from safetensors.torch import save_file
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    hf = dict(cfg)
    hf.update({"architectures": ["LlamaForCausalLM"], "model_type": "llama", "torch_dtype": "bfloat16", "hidden_act": "silu",
               "bos_token_id": 1, "eos_token_id": 2})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(hf, f)
    tok = Tokenizer(WordLevel({"<unk>": 0, "<s>": 1, "</s>": 2, "a": 3}, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "bos_token": "<s>", "eos_token": "</s>"}, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))


def run_reference(name: str, out_dir: str) -> None:
    from cpmcu.llm import LLM                         # the reference's class

    cfg, seed = CONFIGS[name], SEEDS[name]
    ids = make_tokens(cfg, seed)
    folder = tempfile.mkdtemp(prefix=f"cpmcu_golden_{name}_")
    write_folder(folder, cfg, make_weights(cfg, seed))
    llm = LLM(folder, memory_limit=0.05, chunk_length=32, dtype=torch.bfloat16, cuda_graph=False)
    llm.init_storage()
    with torch.no_grad():
        llm._load_from_ckpt(folder)
        d = cfg["head_dim"]
        inv_freq = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        llm._load("model.rotary_emb.inv_freq", inv_freq, dtype=torch.float32)
    dev_ids = torch.tensor(ids, dtype=torch.int32, device="cuda")
    rows, positions = [], []
    for n in PREFIXES:                                # every call starts a sequence at position 0
        logits = llm.prefill(dev_ids[:n], torch.arange(n, dtype=torch.int32, device="cuda"))
        rows.append(logits[0].float().cpu())
        positions.append(n - 1)
    for i in range(DECODED):                          # goes on from the last prompt (PROMPT tokens)
        at = PROMPT + i
        logits = llm.decode(dev_ids[at:at + 1], torch.tensor([at], dtype=torch.int32, device="cuda"),
                            torch.tensor([at], dtype=torch.int32, device="cuda"))
        rows.append(logits[0].float().cpu())
        positions.append(at)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, f"reference_{name}.npz"), config=json.dumps(cfg), seed=seed,
                        ids=np.array(ids, dtype=np.int32), positions=np.array(positions, dtype=np.int32),
                        logits=torch.stack(rows).numpy().astype(np.float32))
    print(f"[golden] {name}: {len(rows)} rows of {cfg['vocab_size']} logits, largest |logit| {float(torch.stack(rows).abs().max()):.3f}")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--only", default=None, help="one configuration's name")
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    # one process per model: the reference keeps one model per process (its storage is a process-wide pool)
    if a.only:
        run_reference(a.only, a.out)
        return 0
    import subprocess
    for name in CONFIGS:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--out", a.out, "--only", name])
        if r.returncode != 0:
            return r.returncode
    return 0


if __name__ == "__main__":
    sys.exit(main())
