#!/usr/bin/env python3
"""Benchmark: decode tokens/s (batch 1, 8, 64) and prefill tokens/s (2,048 tokens) of a
MiniCPM4-8B-sized model with random bf16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run is batch 8 with the
sequences ending at the context length of 4,096 tokens.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# MiniCPM4-8B layer sizes; random weights N(0, 0.02), seed 2; bf16.
MODEL = {
    "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 16384, "vocab_size": 73448,
    "rope_theta": 10000.0, "max_position_embeddings": 65536, "rms_norm_eps": 1e-6,
    "scale_emb": 12, "dim_model_base": 256, "scale_depth": 1.4, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# MiniCPM4-0.5B layer sizes; random weights seed 3; tied head.
MODEL_HALF_B = dict(MODEL, num_hidden_layers=24, hidden_size=1024, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=64, intermediate_size=4096, tie_word_embeddings=True)
# InfLLM-v2 knobs of the long-context workload (8B sizes).
SPARSE_8B = {"kernel_size": 32, "kernel_stride": 16, "block_size": 64, "init_blocks": 1, "topk": 64,
             "window_size": 2048, "dense_len": 8192}
FULL_LAYERS = 32
CONTEXT = 4096
PREFILL_TOKENS = 2048
SEED = 2
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def long_factors(n: int) -> list:
    import torch
    g = torch.Generator().manual_seed(SEED)
    return sorted((1.0 + 39.0 * torch.rand(n, generator=g)).tolist())


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as f:
            data = json.load(f)
        if "hbm_gbs" in data and "bf16_tflops" in data:
            out = {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in data:
                out["bf16_tflops_sustained"] = float(data["bf16_tflops_sustained"])
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for name, v in zip(names, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm(steps: int, warmup: int) -> int:
    """Runs the unmodified reference, installed under baseline/_ref, through its own Python API in a process of
    its own (baseline/run_reference.py; nothing of this package is on that path) and passes its JSON line on.
    The install: a copy of the reference with its empty ``src/cutlass`` submodule folder filled from the CUTLASS
    header tree that ships with an installed package, built with CPMCU_CUDA_ARCH=100 CPMCU_DTYPE=bf16."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "cpmcu")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference (pip install --no-index --no-build-isolation "
                          "--target baseline/_ref of a copy of the reference whose src/cutlass holds CUTLASS headers)"}))
        return 0
    cfgd = dict(MODEL)
    cfgd["rope_scaling"] = {"rope_type": "longrope", "long_factor": long_factors(64), "short_factor": [1.0] * 64,
                            "original_max_position_embeddings": 32768}
    env = dict(os.environ, PYTHONPATH=ref + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "run_reference.py"), "--model-json", json.dumps(cfgd),
           "--steps", str(steps), "--warmup", str(max(3, warmup)), "--context", str(CONTEXT),
           "--prefill-tokens", str(PREFILL_TOKENS), "--seed", str(SEED)]
    try:
        p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd=tempfile.gettempdir())
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference run did not end within 1500 s"}))
        return 0
    line = next((l for l in reversed(p.stdout.splitlines()) if l.startswith("{") and '"impl"' in l), None)
    if p.returncode != 0 or line is None:
        err = [l.strip() for l in (p.stderr + "\n" + p.stdout).splitlines() if l.strip() and not l.startswith("{")]
        picked = [l for l in err if "error" in l.lower() or "Error" in l or "Signal" in l][-3:] or err[-2:]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference run failed (exit {p.returncode}): "
                          + (" | ".join(picked)[:400] if picked else "no output")}))
        sys.stderr.write(p.stderr[-6000:])
        return 0
    print(line)
    return 0


def build_engine(n_layers: int, max_tokens: int, max_batch: int, model: dict = None, seed: int = SEED,
                 max_seq_tokens: int = None, chunk_tokens: int = None, sparse: dict = None):
    import torch
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.engine.storage import make_storage
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    cfgd = dict(model or MODEL, num_hidden_layers=n_layers)
    half = cfgd["head_dim"] // 2
    cfgd["rope_scaling"] = {"rope_type": "longrope", "long_factor": long_factors(half), "short_factor": [1.0] * half,
                            "original_max_position_embeddings": 32768}
    if sparse:
        cfgd["sparse_config"] = dict(sparse)
    arch = architecture("MiniCPMForCausalLM")
    cfg = arch.config_class.from_dict(cfgd)
    # the residual scale of the full depth, whatever number of layers is built
    model = build_model(arch, cfg, torch.bfloat16, "cuda:0")
    chunk = chunk_tokens or PREFILL_TOKENS
    # one arena: weights, step workspace, per-sequence state and the key-value pages (as the Python entry point does)
    if os.environ.get("CPMCU_BENCH_ARENA", "1") == "0":              # for comparisons: every tensor from torch's allocator
        from cpmcu_b200.cache import Cache
        model.load_weights(random_tensors(model.weight_specs(), seed, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0"))
        cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=torch.bfloat16, device="cuda:0",
                      n_slots=max_batch + 2, max_seq_tokens=max_seq_tokens or CONTEXT + 64, max_step_tokens=chunk)
        return cfg, model, cache, Stepper(model, cache, chunk_tokens=chunk, graph_prompts=True)
    storage = make_storage(model, chunk, max_batch, max_tokens=max_tokens, max_seq_tokens=max_seq_tokens or CONTEXT + 64,
                           n_slots=max_batch + 2)
    model.load_weights(random_tensors(model.weight_specs(), seed, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0"))
    torch.cuda.empty_cache()                                         # the loader's tensors: their copies live in the arena
    return cfg, model, storage.cache, Stepper(model, storage.cache, chunk_tokens=chunk, graph_prompts=True)


def random_prompt(vocab: int, n: int, seed: int) -> list:
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def time_decode(stepper, batch: int, steps: int, warmup: int, vocab: int, sample_clocks: bool = False,
                context: int = None):
    """Sequences are prefilled so that the timed steps end at the context length; returns
    (ms per step, clocks, launches in the timed region, bytes of cache read per step)."""
    import torch
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.engine.decode import DecodeRunner
    from cpmcu_b200.ops import library
    from cpmcu_b200.sampling import SamplingParams

    context = context or CONTEXT
    start_len = context - steps - warmup - 1
    slots = stepper.open(batch)
    first = []
    for i, s in enumerate(slots):                       # one prompt per step keeps the workspace small
        out = stepper.step([SequenceStep(s, random_prompt(vocab, start_len, 100 + i), [start_len - 1])])
        first.append(int(out.argmax(dim=-1)[0]))
    runner = DecodeRunner(stepper, use_graph=True, seed=SEED)
    runner.start(slots, first, list(range(batch)), [1] * batch, [SamplingParams()] * batch)
    runner.step()
    for _ in range(max(0, warmup - 1)):
        runner.step()
    torch.cuda.synchronize()
    sampler = ClockSampler()
    if sample_clocks:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        runner.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    clocks = sampler.stop() if sample_clocks else None
    mean_ctx = context - 1 - steps / 2
    cache_bytes = sum(stepper.model.blocks[e.layer].mixer.cache_bytes_read(int(mean_ctx)) for e in stepper.model.schedule) * batch
    launches = runner.launches_per_graph * steps
    for s in slots:
        stepper.close(s)
    stepper.close(runner.pad_slot)
    return ms, clocks, launches, cache_bytes


def time_prefill(stepper, cfg, reps: int = 3):
    import torch
    from cpmcu_b200.engine import SequenceStep

    times = []
    for r in range(reps + 1):
        ids = random_prompt(cfg.vocab_size, PREFILL_TOKENS, 500 + r)
        slot = stepper.open(1)[0]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stepper.step([SequenceStep(slot, ids, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if r > 0:
            times.append(e0.elapsed_time(e1))
        stepper.close(slot)
    return statistics.median(times)


def prefill_flops(cfg, n_layers: int, tokens: int) -> float:
    h, d = cfg.hidden_size, cfg.head_dim
    per_layer = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * h + cfg.num_attention_heads * d * h \
        + 3 * cfg.intermediate_size * h
    gemm = 2.0 * tokens * per_layer * n_layers + 2.0 * cfg.vocab_size * h
    attn = 4.0 * cfg.num_attention_heads * d * tokens * tokens / 2 * n_layers
    return gemm + attn


def time_e2e(cfg, stepper, steps: int, batch: int):
    """The same decode metric through the Python entry point's loop: host token lists in,
    host token lists out, one device-to-host read of the sampled tokens per step."""
    import torch
    from cpmcu_b200.engine.backend import EngineBackend
    from cpmcu_b200.engine.generate import Request, run_requests
    from cpmcu_b200.sampling import SamplingParams

    backend = EngineBackend(stepper, max_batch=batch, use_graph=True, seed=SEED)
    n_new = steps + 1
    prompts = [random_prompt(cfg.vocab_size, CONTEXT - n_new, 900 + i) for i in range(batch)]
    reqs = [Request(p, n_new, SamplingParams(), (), key=i) for i, p in enumerate(prompts)]
    run_requests(backend, [Request(p[:64], 4, SamplingParams(), (), key=i) for i, p in enumerate(prompts)],
                 sync=torch.cuda.synchronize)                       # warm-up: graph capture
    h0, d0 = backend.h2d_bytes, backend.d2h_bytes
    results, stats = run_requests(backend, reqs, sync=torch.cuda.synchronize)
    assert all(len(r.tokens) == n_new for r in results)
    decode_steps = max(1, stats.decode_steps)
    prompt_bytes = 4 * sum(len(p) for p in prompts)
    return {
        "value": batch * decode_steps / stats.decode_time, "unit": "tokens/s",
        "h2d_bytes_per_step": (backend.h2d_bytes - h0 - prompt_bytes) / decode_steps,
        "d2h_bytes_per_step": (backend.d2h_bytes - d0) / (decode_steps + 1),
        "prefill_tokens_per_s": stats.prompt_tokens / stats.prefill_time,
    }


def loop_prefill(stepper, prompts, max_batch: int):
    """Prompts of one batch through the generation loop's backend (chunked as the stepper is set up), one new token
    each; returns (tokens per second, milliseconds)."""
    import torch
    from cpmcu_b200.engine.backend import EngineBackend
    from cpmcu_b200.engine.generate import Request, run_requests
    from cpmcu_b200.sampling import SamplingParams

    backend = EngineBackend(stepper, max_batch=max_batch, use_graph=True, seed=SEED)
    reqs = [Request(p, 1, SamplingParams(), (), key=i) for i, p in enumerate(prompts)]
    run_requests(backend, [Request(p[:64], 1, SamplingParams(), (), key=i) for i, p in enumerate(prompts)],
                 sync=torch.cuda.synchronize)                                   # warm-up
    best = None
    for _ in range(2):
        _, stats = run_requests(backend, reqs, sync=torch.cuda.synchronize)
        best = stats.prefill_time if best is None else min(best, stats.prefill_time)
    stepper.close(backend.runner.pad_slot)
    return sum(len(p) for p in prompts) / best, best * 1e3


def workload_half_b(steps: int, warmup: int) -> int:
    """MiniCPM4-0.5B layer sizes: 64 prompts of unequal lengths (uniform in [64, 2048]) prefilled in chunks of 512
    packed tokens, and decode steps of the 64 sequences that end at a context of 8,192 tokens."""
    import torch

    batch, context, chunk = 64, 8192, 512
    pk = peaks()
    cfg, model, cache, stepper = build_engine(MODEL_HALF_B["num_hidden_layers"], batch * (context + 64) + 128, batch,
                                              model=MODEL_HALF_B, seed=3, max_seq_tokens=context + 64, chunk_tokens=2048)
    stepper.chunk_tokens = chunk                                                # the workload's prompts: chunks of 512
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(64, 2049, (batch,), generator=g).tolist()
    prompts = [random_prompt(cfg.vocab_size, n, 300 + i) for i, n in enumerate(lens)]
    prefill_tps, prefill_ms = loop_prefill(stepper, prompts, batch)
    stepper.chunk_tokens = 2048                                                 # the long warm-up prompts in larger pieces
    ms, clocks, launches, cache_bytes = time_decode(stepper, batch, steps, warmup, cfg.vocab_size, True, context=context)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "workload": "half_b", "metric": "decode tokens/s (MiniCPM4-0.5B sizes, bf16, batch 64, context 8192)",
        "value": batch * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 3",
        "config": {"model": "MiniCPM4-0.5B sizes", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": True, "global_batch": batch,
                   "seq_len": context, "prompt_lengths": "uniform in [64, 2048]", "chunk_length": chunk, "cuda_graph": True,
                   "peaks": pk["source"]},
        "prefill": {"value": prefill_tps, "tokens": sum(lens), "ms": prefill_ms, "through": "generation loop"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "weight_bytes": weight_bytes, "cache_bytes": cache_bytes},
        "clocks": clocks, "gpu_launches": launches,
    }))
    return 0


def workload_sparse8b(steps: int, warmup: int, layers: int) -> int:
    """MiniCPM4-8B layer sizes with InfLLM-v2 block-sparse attention: prompts of 16,384 and 30,000 tokens in one
    batch, prefilled in chunks of 2,048 packed tokens through the generation loop, then decode steps of the two
    sequences under a CUDA graph."""
    import torch
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.engine.decode import DecodeRunner
    from cpmcu_b200.sampling import SamplingParams

    lens, context = [16384, 30000], 32768
    pk = peaks()
    cfg, model, cache, stepper = build_engine(layers, 3 * context + 256, 2, seed=4, max_seq_tokens=context + 64,
                                              chunk_tokens=2048, sparse=SPARSE_8B)
    prompts = [random_prompt(cfg.vocab_size, n, 40 + i) for i, n in enumerate(lens)]
    prefill_tps, prefill_ms = loop_prefill(stepper, prompts, 2)
    stepper.ops.raise_on_kernel_error()
    slots = stepper.open(2)
    first = []
    for s_, p_ in zip(slots, prompts):
        out = stepper.step([SequenceStep(s_, p_, [len(p_) - 1])])
        first.append(int(out.argmax(dim=-1)[0]))
    runner = DecodeRunner(stepper, use_graph=True, seed=SEED)
    runner.start(slots, first, [0, 1], [1, 1], [SamplingParams()] * 2)
    for _ in range(max(3, warmup)):
        runner.step()
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        runner.step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    stepper.ops.raise_on_kernel_error()
    ms = e0.elapsed_time(e1) / steps
    mean_ctx = [n + max(3, warmup) + steps // 2 for n in lens]
    cache_bytes = sum(stepper.model.blocks[e.layer].mixer.cache_bytes_read(c) for e in stepper.model.schedule for c in mean_ctx)
    dense_bytes = sum(2 * c * cfg.num_key_value_heads * cfg.head_dim * 2 * layers for c in mean_ctx)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "workload": "sparse8b", "metric": "decode ms/step and prefill tokens/s (MiniCPM4-8B sizes, InfLLM-v2, batch 2, context 32768)",
        "value": 2 * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": max(3, warmup),
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 4",
        "config": {"model": "MiniCPM4-8B sizes", "layers": layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": 2, "seq_len": context,
                   "prompt_lengths": "16384 and 30000", "chunk_length": 2048, "attention": "InfLLM-v2 32/16/64/1/64/2048/8192",
                   "cuda_graph": True, "peaks": pk["source"]},
        "prefill": {"value": prefill_tps, "tokens": sum(lens), "ms": prefill_ms, "through": "generation loop"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "weight_bytes": weight_bytes, "cache_bytes": cache_bytes,
                     "cache_bytes_if_dense": dense_bytes},
        "clocks": clocks, "gpu_launches": runner.launches_per_graph * steps,
    }))
    return 0


def step_launches(name: str, batch: int, ctx: int, layers: int, reps: int, workload: str = "dense8b") -> int:
    """A few eager steps of a model with few layers of a workload's sizes, one kernel launch after the other, for
    a profiler's launch list: decode_step = one token for each of ``batch`` sequences that hold ``ctx`` tokens;
    prefill_step = a prompt of ``ctx`` tokens."""
    import torch
    from cpmcu_b200.engine import SequenceStep

    global CONTEXT
    CONTEXT = max(CONTEXT, ctx + 64)
    cfg, model, cache, stepper = build_engine(layers, batch * (ctx + 128) + 128, batch,
                                              model=MODEL_HALF_B if workload == "half_b" else MODEL,
                                              sparse=SPARSE_8B if workload == "sparse8b" else None)
    if name == "decode_step":
        slots = stepper.open(batch)
        for i, s in enumerate(slots):
            stepper.step([SequenceStep(s, random_prompt(cfg.vocab_size, ctx, i), [])])
        torch.cuda.synchronize()
        for _ in range(max(1, reps)):
            out = stepper.step([SequenceStep(s, [5], [0]) for s in slots])
            torch.cuda.synchronize()
    else:
        for r in range(max(1, reps)):
            slot = stepper.open(1)[0]
            out = stepper.step([SequenceStep(slot, random_prompt(cfg.vocab_size, ctx, r), [ctx - 1])])
            torch.cuda.synchronize()
            stepper.close(slot)
    print(json.dumps({"kernel": name, "workload": workload, "batch": batch, "ctx": ctx, "layers": layers, "logits": list(out.shape)}))
    return 0


def kernel_bench(name: str, batch: int, ctx: int, rows: int, n: int, k: int, reps: int) -> int:
    """One kernel alone at the benchmark's shapes, timed inside a CUDA graph with rotating
    buffers larger than L2 (also the target of the ncu captures under profiles/)."""
    import math
    import torch
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import PREFILL_TILE_ROWS, Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops, dev = Ops(torch.bfloat16, "cuda:0"), "cuda:0"
    heads, kv, d = MODEL["num_attention_heads"], MODEL["num_key_value_heads"], MODEL["head_dim"]

    def timed(fn, n_inner):
        fn(0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n_inner):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * n_inner)

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    out = {"kernel": name}
    if name == "skinny_gemm":
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
        us = timed(lambda i: ops.linear(x, ws[i % copies]), copies * 2)
        out.update(rows=rows, n=n, k=k, us=us, gbs=n * k * 2 / 1e3 / us)
    elif name == "decode_attention":
        lanes = max(2, int(400e6 // (batch * ctx * kv * d * 4)) + 1)
        cache = Cache([CacheNeeds(kv_heads=kv, head_dim=d)] * lanes, max_tokens=batch * (ctx + 64), dtype=torch.bfloat16,
                      device=dev, n_slots=batch + 1, max_seq_tokens=ctx + 64)
        slots = cache.open_sequences(batch)
        for s_ in slots:
            cache.reserve(s_, ctx)
        cache.sync()
        for lane in cache.lanes:
            lane.k.normal_()
            lane.v.normal_()
        q = torch.randn(batch, heads, d, device=dev, dtype=torch.bfloat16)
        kv_len, sl = i32([ctx] * batch), i32(slots)
        us = timed(lambda i: ops.decode_attention(q, cache.lane(i % lanes).k, cache.lane(i % lanes).v, kv_len, sl,
                                                  cache.lane(0).page_table, kv, 1 / math.sqrt(d)), lanes * 2)
        out.update(batch=batch, ctx=ctx, us=us, gbs=batch * ctx * kv * d * 4 / 1e3 / us)
    elif name in ("prefill_attention", "prefill_attention_mma"):
        cache = Cache([CacheNeeds(kv_heads=kv, head_dim=d)], max_tokens=ctx + 64, dtype=torch.bfloat16, device=dev, n_slots=2)
        slot = cache.open_sequence()
        cache.reserve(slot, ctx)
        cache.sync()
        cache.lane(0).k.normal_()
        cache.lane(0).v.normal_()
        q = torch.randn(ctx, heads, d, device=dev, dtype=torch.bfloat16)
        n_tiles = (ctx + PREFILL_TILE_ROWS - 1) // PREFILL_TILE_ROWS
        tiles = (i32([0] * n_tiles), i32(list(range(0, ctx, PREFILL_TILE_ROWS))), n_tiles)
        cu, kv_len, sl = i32([0, ctx]), i32([ctx]), i32([slot])
        fn = ops.prefill_attention if name == "prefill_attention_mma" else ops.prefill_attention_tcgen05
        us = timed(lambda i: fn(q, cache.lane(0).k, cache.lane(0).v, tiles, cu, kv_len, sl,
                                cache.lane(0).page_table, kv, 1 / math.sqrt(d)), 4)
        out.update(tokens=ctx, us=us, tflops=4 * heads * d * ctx * ctx / 2 / us / 1e6,
                   error_code=ops.attention_tcgen05_error())
    elif name == "gemm_tcgen05":
        # the gated gate_up product of a prompt chunk: rows x k times (n x k)^T, silu(gate) * up in the epilogue
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
        us = timed(lambda i: ops.linear_tcgen05(x, ws[i % copies], gated=True), copies * 2)
        out.update(rows=rows, n=n, k=k, us=us, tflops=2.0 * rows * n * k / us / 1e6, error_code=ops.tcgen05_error())
    else:
        print(f"unknown kernel '{name}'; known: skinny_gemm, decode_attention, prefill_attention, prefill_attention_mma, gemm_tcgen05")
        return 2
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="layers built (the full model has 32)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--workload", default="dense8b", choices=["dense8b", "half_b", "sparse8b"],
                    help="dense8b: the headline line (8B sizes, batch 8, context 4096); half_b: 0.5B sizes, batch 64, prompts "
                         "uniform in [64, 2048] chunked at 512, decode at context 8192 (256 steps by default); sparse8b: 8B "
                         "sizes with InfLLM-v2, prompts of 16384 and 30000 tokens chunked at 2048, then decode steps")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the e2e run")
    ap.add_argument("--kernel", default=None, help="time one kernel alone: skinny_gemm, decode_attention, prefill_attention (tcgen05), prefill_attention_mma, gemm_tcgen05; or run eager steps of a 2-layer model for a launch list: decode_step, prefill_step")
    ap.add_argument("--ctx", type=int, default=CONTEXT, help="--kernel: cached tokens per sequence (or prompt tokens)")
    ap.add_argument("--rows", type=int, default=8, help="--kernel skinny_gemm / gemm_tcgen05: rows of the activation")
    ap.add_argument("--n", type=int, default=4096, help="--kernel skinny_gemm: output features")
    ap.add_argument("--k", type=int, default=4096, help="--kernel skinny_gemm: input features")
    ap.add_argument("--reps", type=int, default=5, help="--kernel: graph replays that are timed")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a.steps, a.warmup)
    if a.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus must be 1")
        return 2
    if a.kernel in ("decode_step", "prefill_step"):
        return step_launches(a.kernel, a.batch, a.ctx, a.layers if a.layers != FULL_LAYERS else 2, a.reps, a.workload)
    if a.workload == "half_b":
        return workload_half_b(a.steps if a.steps != 128 else 256, max(3, a.warmup))
    if a.workload == "sparse8b":
        return workload_sparse8b(a.steps, a.warmup, a.layers)
    if a.kernel:
        return kernel_bench(a.kernel, a.batch, a.ctx, a.rows, a.n, a.k, a.reps)
    a.warmup = max(3, a.warmup)
    import torch
    from cpmcu_b200.ops import library

    pk = peaks()
    max_batch = a.batch if a.no_points else max(64, a.batch)
    cfg, model, cache, stepper = build_engine(a.layers, max_batch * (CONTEXT + 64) + 128, max_batch)
    weight_bytes = model.weight_bytes_per_step()

    ms, clocks, launches, cache_bytes = time_decode(stepper, a.batch, a.steps, a.warmup, cfg.vocab_size, True)
    value = a.batch * 1000.0 / ms
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9

    pre_ms = time_prefill(stepper, cfg)
    flops = prefill_flops(cfg, a.layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}
    if "bf16_tflops_sustained" in pk:       # the step is 32 layers long: the peak under the power cap, beside the burst peak
        prefill["frac_sustained"] = flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12)

    points, e2e = {}, None
    if not a.no_points:
        for b in (1, 64):
            pms, _, _, _ = time_decode(stepper, b, min(a.steps, 64), a.warmup, cfg.vocab_size)
            points[f"decode_b{b}"] = b * 1000.0 / pms
        e2e = time_e2e(cfg, stepper, a.steps, a.batch)

    line = {
        "metric": "decode tokens/s (MiniCPM4-8B sizes, bf16, batch 8, context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 2",
        "impl": "ours",
        "config": {
            "model": "MiniCPM4-8B sizes", "layers": a.layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": a.batch,
            "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "rope": "longrope", "attention": "dense", "l2": "inputs larger than L2 (weights read per step)",
            "peaks": pk["source"], "cuda_graph": True,
        },
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "clocks": clocks,
        "gpu_launches": launches,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
