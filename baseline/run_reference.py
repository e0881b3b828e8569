#!/usr/bin/env python3
"""Times the unmodified reference (OpenBMB/CPM.cu, installed under baseline/_ref) on the
benchmark's model sizes through its own Python API: ``cpmcu.llm.LLM`` with ``init_storage``,
``load_from_hf``/``_load``, ``prefill``, ``decode`` and ``generate``.

Nothing of cpmcu_b200 is imported here.  The reference runs one sequence at a time, so the
decode figure is for batch 1.  The model folder is made in a temporary place: a config.json
with the benchmark's sizes (as a ``llama`` configuration carrying MiniCPM's scale keys, which
is how the reference reads them: cpmcu/llm.py:62-69), a word-level tokenizer.json (the
reference's constructor loads a tokenizer), and a safetensors file with the final norm only;
all matrices are random tensors made here and handed to the reference's own ``_load`` (one
random tensor per shape, reused for every layer: the values do not matter for the timing).

Prints one JSON line.  Run by ``bench.py --impl reference``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time


def write_folder(folder: str, m: dict, rope_scaling) -> None:
    from safetensors.torch import save_file
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    import torch

    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": m["vocab_size"], "hidden_size": m["hidden_size"], "intermediate_size": m["intermediate_size"],
        "num_hidden_layers": m["num_hidden_layers"], "num_attention_heads": m["num_attention_heads"],
        "num_key_value_heads": m["num_key_value_heads"], "head_dim": m["head_dim"], "rms_norm_eps": m["rms_norm_eps"],
        "rope_theta": m["rope_theta"], "max_position_embeddings": m["max_position_embeddings"],
        "tie_word_embeddings": False, "torch_dtype": "bfloat16", "hidden_act": "silu",
        "scale_emb": m["scale_emb"], "dim_model_base": m["dim_model_base"], "scale_depth": m["scale_depth"],
        "bos_token_id": 1, "eos_token_id": 2,
    }
    if rope_scaling is not None:
        cfg["rope_scaling"] = rope_scaling
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    tok = Tokenizer(WordLevel({"<unk>": 0, "<s>": 1, "</s>": 2, "a": 3}, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "bos_token": "<s>",
                   "eos_token": "</s>"}, f)
    save_file({"model.norm.weight": torch.ones(m["hidden_size"], dtype=torch.bfloat16)},
              os.path.join(folder, "model.safetensors"))


def stage(what: str) -> None:
    """A line on standard error before every stage, so that a crash inside the reference's native code shows where."""
    print(f"[run_reference] {what}", file=sys.stderr, flush=True)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-json", required=True, help="the benchmark's model sizes, as JSON")
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=2)
    a = ap.parse_args()
    m = json.loads(a.model_json)

    import torch
    from cpmcu.llm import LLM                                 # the reference's class, from baseline/_ref

    notes = []
    tmp = tempfile.mkdtemp(prefix="cpmcu_ref_model_")

    def rope_call_works() -> bool:
        """The call cpmcu/llm.py:181-192 makes for the rotary table, tried on the folder before the reference
        takes its memory pool (a second attempt after that would find no memory left)."""
        try:
            from transformers import AutoConfig
            from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
            cfg = AutoConfig.from_pretrained(tmp, trust_remote_code=True)
            rs = getattr(cfg, "rope_scaling", None)
            rope_type = rs.get("rope_type", rs.get("type")) if rs else "default"
            if rope_type == "longrope" and not hasattr(cfg.rope_scaling, "factor"):
                cfg.rope_scaling["factor"] = 1.0
            ROPE_INIT_FUNCTIONS[rope_type](cfg, "cpu", seq_len=a.context)
            return True
        except Exception as e:
            notes.append(f"rotary table call failed ({type(e).__name__}: {str(e)[:100]})")
            return False

    stock_rope = False
    for rs in ([m.get("rope_scaling"), None] if m.get("rope_scaling") else [None]):
        write_folder(tmp, m, rs)
        if rope_call_works():
            stock_rope = True
            if rs is None and m.get("rope_scaling"):
                notes.append("plain rotary factors (the long factors change no timing)")
            break
    stage("constructing cpmcu.llm.LLM")
    llm = LLM(tmp, memory_limit=0.8, chunk_length=a.prefill_tokens, dtype=torch.bfloat16, cuda_graph=True)
    if os.environ.get("CPMCU_BT"):                            # a native backtrace on a crash, for finding where it is
        import ctypes
        ctypes.CDLL(os.environ["CPMCU_BT"]).install()
    stage("init_storage")
    llm.init_storage()
    stage(f"max_total_length {llm.max_total_length}; load_from_hf")
    if stock_rope:
        llm.load_from_hf()                                    # the final norm from the file, then the rotary table
    else:
        notes.append("rotary table 1/theta^(2c/d) handed to LLM._load instead of load_from_hf's own call")
        with torch.no_grad():
            llm._load_from_ckpt(tmp)
            inv = 1.0 / (m["rope_theta"] ** (torch.arange(0, m["head_dim"], 2, dtype=torch.float32) / m["head_dim"]))
            llm._load("model.rotary_emb.inv_freq", inv, dtype=torch.float32)

    g = torch.Generator().manual_seed(a.seed)
    H, I, V = m["hidden_size"], m["intermediate_size"], m["vocab_size"]
    nh, nkv, d = m["num_attention_heads"], m["num_key_value_heads"], m["head_dim"]
    shapes = {"q_proj": (nh * d, H), "k_proj": (nkv * d, H), "v_proj": (nkv * d, H), "o_proj": (H, nh * d),
              "gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
    rand = {k: (torch.randn(s, generator=g) * 0.02).to(torch.bfloat16) for k, s in shapes.items()}
    norm = (1.0 + 0.02 * torch.randn(H, generator=g)).to(torch.bfloat16)
    stage("loading random matrices through LLM._load")
    with torch.no_grad():
        llm._load("model.embed_tokens.weight", (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16))
        llm._load("lm_head.weight", (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16))
        for layer in range(m["num_hidden_layers"]):
            p = f"model.layers.{layer}."
            llm._load(p + "input_layernorm.weight", norm)
            llm._load(p + "post_attention_layernorm.weight", norm)
            for k in ("q_proj", "k_proj", "v_proj", "o_proj"):
                llm._load(p + f"self_attn.{k}.weight", rand[k])
            for k in ("gate_proj", "up_proj", "down_proj"):
                llm._load(p + f"mlp.{k}.weight", rand[k])
    torch.cuda.synchronize()

    def ids(n, seed):
        gg = torch.Generator().manual_seed(seed)
        return torch.randint(0, V, (n,), generator=gg, dtype=torch.int32).cuda()

    def event_ms(fn):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    # prefill of one prompt, last-row logits (the reference's prefill), median of three after a warm-up
    stage("prefill")
    P = a.prefill_tokens
    pos = torch.arange(P, dtype=torch.int32, device="cuda")
    times = [event_ms(lambda r=r: llm.prefill(ids(P, 500 + r), pos)) for r in range(4)][1:]
    prefill_ms = statistics.median(times)

    # decode, one sequence: the timed steps end at the context length
    stage("decode")
    start = a.context - a.steps - a.warmup - 1
    llm.prefill(ids(start, 100), torch.arange(start, dtype=torch.int32, device="cuda"))
    tok = torch.tensor([5], dtype=torch.int32, device="cuda")
    p1 = torch.tensor([0], dtype=torch.int32, device="cuda")
    cl = torch.tensor([0], dtype=torch.int32, device="cuda")
    at = [start]

    def steps(n):
        for _ in range(n):
            p1[0] = at[0]
            cl[0] = at[0]
            logits = llm.decode(tok, p1, cl)
            tok[0] = logits[0].argmax(dim=-1)
            at[0] += 1

    steps(a.warmup)
    decode_ms = event_ms(lambda: steps(a.steps)) / a.steps

    # end to end: the reference's own generate(), host ids in, host tokens out
    stage("generate")
    prompt = ids(a.context - a.steps - 1, 900)
    llm.generate(prompt[:64], generation_length=4)
    tokens, decode_time, prefill_time = llm.generate(prompt, generation_length=a.steps + 1, terminators=[])
    e2e = (len(tokens) - 1) / decode_time

    print(json.dumps({
        "impl": "reference", "metric": "decode tokens/s (MiniCPM4-8B sizes, bf16, batch 1, context %d)" % a.context,
        "value": 1000.0 / decode_ms, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": decode_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights N(0,0.02), one tensor per shape reused for every layer",
        "config": {"model": "MiniCPM4-8B sizes", "layers": m["num_hidden_layers"], "hidden": H, "heads": nh, "kv_heads": nkv,
                   "head_dim": d, "intermediate": I, "vocab": V, "global_batch": 1, "seq_len": a.context,
                   "prefill_tokens": P, "parallelism": "single GPU", "attention": "dense", "cuda_graph": True,
                   "note": "the reference runs one sequence at a time: batch 1"},
        "prefill": {"value": P / (prefill_ms * 1e-3), "tokens": P, "ms": prefill_ms},
        "points": {"decode_b1": 1000.0 / decode_ms},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4,
                "prefill_tokens_per_s": prompt.numel() / prefill_time},
        "notes": notes,
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
