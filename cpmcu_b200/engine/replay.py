"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
the same :class:`Stepper`, cache and kernels that generation uses.  Steps arrive on
standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step with wanted places the fp32 logits [wanted, vocab] go to ``<out>/<step>.f32``
(little-endian), in the order of the entries and of each ``want``.  After every step a
line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, IO, Optional

import torch

from ..cache import Cache, pages_for, PAGE_TOKENS
from ..loading import load_model, parse_dtype
from .step import SequenceStep, Stepper


def run(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stdin: IO[str], stdout: IO[str],
        device: str = "cuda:0", chunk_tokens: int = 2048) -> int:
    os.makedirs(out_dir, exist_ok=True)
    _, config, model = load_model(model_dir, parse_dtype(dtype), device)
    cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=model.ops.dtype, device=device,
                  max_step_tokens=chunk_tokens)
    stepper = Stepper(model, cache, chunk_tokens=chunk_tokens)
    slots: Dict[str, int] = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step_no = msg["step"]
        batch = []
        for entry in msg.get("entries", []):
            rid = str(entry["id"])
            if rid not in slots:
                slots[rid] = stepper.open(1)[0]
            batch.append(SequenceStep(slots[rid], entry["tokens"], entry.get("want", [])))
        logits = stepper.step(batch)
        if logits is not None:
            data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(out_dir, f".{step_no}.f32.tmp")
            data.tofile(tmp)
            os.replace(tmp, os.path.join(out_dir, f"{step_no}.f32"))
        else:
            torch.cuda.synchronize()
        stepper.ops.raise_on_kernel_error()
        for rid in msg.get("end", []):
            rid = str(rid)
            if rid in slots:
                stepper.close(slots.pop(rid))
        stdout.write(f"done {step_no}\n")
        stdout.flush()
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder the logits files are written to")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache")
    p.add_argument("--chunk-tokens", type=int, default=2048, help="most packed tokens one forward pass takes")
    p.add_argument("--device", default="cuda:0")
    a = p.parse_args(argv)
    return run(a.model, a.dtype, a.out, a.max_tokens, sys.stdin, sys.stdout, a.device, a.chunk_tokens)


if __name__ == "__main__":
    sys.exit(main())
