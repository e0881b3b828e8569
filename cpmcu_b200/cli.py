"""Command line in the manner of ``python -m cpmcu.cli`` (cpmcu/cli.py:304-329,
cpmcu/common/args.py:22-131): the same option names and meanings where the reference
has them; every flag has a ``--kebab-case`` and a ``--snake_case`` spelling.

    python -m cpmcu_b200.cli --model-path DIR --prompt-text "..." --num-generate 64
    python -m cpmcu_b200.cli --model-path DIR --prompt-ids 5,17,3 --temperature 0.8 --random-seed 1

Options the reference has and this library leaves out belong to parts that are not
built (draft models, quantized weights, the per-flag sparse-attention knobs: those come
from the folder's config.json here).  Added: ``--prompt-ids`` (token ids, no tokenizer
needed), ``--top-p``, ``--max-batch``, ``--max-tokens``, ``--plugin`` (a module that registers
parts or an architecture of its own).
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import List, Optional


def str2bool(v):
    if isinstance(v, bool):
        return v
    if v.lower() in ("yes", "true", "t", "y", "1"):
        return True
    if v.lower() in ("no", "false", "f", "n", "0"):
        return False
    raise argparse.ArgumentTypeError("Boolean value expected.")


def create_cli_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="cpmcu_b200.cli", description="cpmcu_b200 command line")
    flag = dict(type=str2bool, nargs="?", const=True)

    g = parser.add_argument_group("Prompt Configuration")
    g.add_argument("--prompt-file", "--prompt_file", type=str, default=None, help="Path to prompt file")
    g.add_argument("--prompt-text", "--prompt_text", type=str, default=None, help="Direct prompt text")
    g.add_argument("--prompt-ids", "--prompt_ids", type=str, default=None, action="append",
                   help="Prompt as comma-separated token ids (may be given several times for a batch)")
    g.add_argument("--use-chat-template", "--use_chat_template", default=True, **flag,
                   help="Use chat template for prompt formatting (default: True)")

    g = parser.add_argument_group("Generation Configuration")
    g.add_argument("--use-stream", "--use_stream", default=True, **flag, help="Use stream generation (default: True)")
    g.add_argument("--num-generate", "--num_generate", type=int, default=1024,
                   help="Number of tokens to generate (default: 1024)")
    g.add_argument("--temperature", "--temp", type=float, default=0.0, help="Temperature (default: 0.0)")
    g.add_argument("--top-p", "--top_p", type=float, default=1.0, help="Nucleus mass kept when sampling (default: 1.0)")
    g.add_argument("--random-seed", "--random_seed", type=int, default=None, help="Random seed")
    g.add_argument("--ignore-eos", "--ignore_eos", default=False, **flag,
                   help="Ignore EOS tokens during generation (default: False)")

    g = parser.add_argument_group("Model Configuration")
    g.add_argument("--model-path", "--model_path", "--model", type=str, required=True,
                   help="Path to the model folder (config.json and safetensors)")
    g.add_argument("--model-type", "--model_type", type=str, default="auto", choices=["auto", "minicpm4"],
                   help="Model type (default: auto = the architecture named in config.json)")
    g.add_argument("--dtype", type=str, default="bfloat16", choices=["bfloat16", "float32"],
                   help="Model dtype (default: bfloat16)")

    g.add_argument("--plugin", type=str, default=None, action="append",
                   help="Module to import before the model is built; it registers parts or an architecture the "
                        "package does not know (may be given several times; also: environment variable CPMCU_PLUGINS)")
    g.add_argument("--random-weights", "--random_weights", type=int, default=None, metavar="SEED",
                   help="Write config.json and model.safetensors with seeded random weights into --model-path "
                        "from the configuration given by --config, then generate from that folder")
    g.add_argument("--config", type=str, default=None, help="config.json for --random-weights")
    g.add_argument("--dense", default=False, **flag,
                   help="Ignore the configuration's sparse_config and attend to all keys (default: False)")

    g = parser.add_argument_group("System Configuration")
    g.add_argument("--cuda-graph", "--cuda_graph", default=True, **flag, help="Use CUDA graph optimization (default: True)")
    g.add_argument("--memory-limit", "--memory_limit", type=float, default=0.9, help="Memory limit (default: 0.9)")
    g.add_argument("--chunk-length", "--chunk_length", type=int, default=2048, help="Chunked prefill size (default: 2048)")
    g.add_argument("--plain-output", "--plain_output", default=False, **flag,
                   help="Use plain text output (default: False; output is always plain here)")
    g.add_argument("--max-batch", "--max_batch", type=int, default=64, help="Most sequences in one batch (default: 64)")
    g.add_argument("--max-tokens", "--max_tokens", type=int, default=None,
                   help="Tokens the cache holds (default: from --memory-limit)")
    return parser


def _load_tokenizer(path: str):
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(path, trust_remote_code=True)
    except Exception as e:  # no tokenizer files, or the package is absent
        return None


def make_prompts(args, tokenizer) -> List[List[int]]:
    """Token ids of the prompts (cpmcu/cli.py:47-79 builds one prompt from text or file)."""
    if args.prompt_ids:
        return [[int(x) for x in s.replace(" ", "").split(",") if x] for s in args.prompt_ids]
    text = args.prompt_text
    if text is None and args.prompt_file:
        with open(args.prompt_file, "r", encoding="utf-8") as f:
            text = f.read()
    if text is None:
        text = "Who are you?"
    if tokenizer is None:
        raise SystemExit("this model folder has no tokenizer; give the prompt as --prompt-ids 1,2,3")
    if args.use_chat_template and getattr(tokenizer, "chat_template", None):
        text = tokenizer.apply_chat_template([{"role": "user", "content": text}], tokenize=False,
                                             add_generation_prompt=True)
    return [list(tokenizer(text, add_special_tokens=False)["input_ids"])]


def write_random_folder(config_path: Optional[str], out_dir: str, seed: int, dtype: str) -> str:
    """The random-weights mode: a model folder from a configuration file and a seed."""
    import json

    from .loading import parse_dtype
    from .models.model import Model
    from .registry import architecture
    from .weights import write_model_folder

    if not config_path:
        raise ValueError("--random-weights needs --config (a config.json to take the sizes from)")
    with open(config_path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    names = raw.get("architectures") or []
    if not names:
        raise ValueError(f"{config_path} names no architecture")
    arch = architecture(names[0])
    config = arch.config_class.from_dict(raw)
    specs = Model(arch.model_spec(config), None).weight_specs()
    folder = write_model_folder(config, specs, out_dir, int(seed), parse_dtype(dtype))
    print(f"[cpmcu_b200] wrote random weights (seed {seed}) to {folder}", file=sys.stderr)
    return folder


def run_generation(args) -> int:
    from .llm import LLM
    from .registry import load_plugins

    if args.plugin:
        load_plugins(args.plugin)
    if args.random_weights is not None:
        write_random_folder(args.config, args.model_path, args.random_weights, args.dtype)
    tokenizer = None if args.prompt_ids else _load_tokenizer(args.model_path)
    llm = LLM(args.model_path, apply_sparse=not args.dense, memory_limit=args.memory_limit, chunk_length=args.chunk_length, dtype=args.dtype,
              cuda_graph=args.cuda_graph, temperature=args.temperature, random_seed=args.random_seed,
              top_p=args.top_p, max_batch=args.max_batch, max_tokens=args.max_tokens)
    llm.tokenizer = tokenizer
    prompts = make_prompts(args, tokenizer)
    terminators = [] if args.ignore_eos else list(llm.model.spec.stop_token_ids)
    if tokenizer is not None and not args.ignore_eos and tokenizer.eos_token_id is not None:
        terminators = sorted(set(terminators) | {int(tokenizer.eos_token_id)})
    max_len = llm.init_storage()
    print(f"[cpmcu_b200] cache holds {llm.cache.max_tokens} tokens, longest sequence {max_len}", file=sys.stderr)
    llm.load_from_hf()

    if args.use_stream and len(prompts) == 1:
        tokens = []
        for item in llm.generate(prompts[0], args.num_generate, terminators, use_stream=True):
            tokens.append(item["token"])
            print(item["text"] if tokenizer else f"{item['token']} ", end="", flush=True)
        print()
        results = [tokens]
    else:
        results = [r.tokens for r in llm.generate_batch(prompts, args.num_generate, terminators)]
        for i, toks in enumerate(results):
            shown = tokenizer.decode(toks, skip_special_tokens=True) if tokenizer else " ".join(map(str, toks))
            print(f"[{i}] {shown}")
    s = llm.last_stats
    if s is not None:
        print(f"prefill length: {s.prompt_tokens}  prefill time: {s.prefill_time:.3f} s  "
              f"prefill tokens/s: {s.prompt_tokens / max(s.prefill_time, 1e-9):.2f}", file=sys.stderr)
        print(f"decode length: {s.generated_tokens}  decode time: {s.decode_time:.3f} s  "
              f"decode tokens/s: {s.generated_tokens / max(s.decode_time, 1e-9):.2f}", file=sys.stderr)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    args = create_cli_parser().parse_args(argv)
    try:
        return run_generation(args)
    except (ValueError, RuntimeError, MemoryError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
