"""The Python entry point, in the manner of the reference's ``cpmcu.llm.LLM``
(cpmcu/llm.py:24-379): construct with a model folder, ``init_storage()``,
``load_from_hf()``, then ``generate()``.

Differences a user will meet: the dtype is bfloat16 or float32 (the reference runs
float16 or bfloat16); prompts may be a batch of unequal lengths; the sparse-attention
knobs come from the folder's config.json, not from arguments; the returned token ids
are Python lists.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Union

import torch

from .cache import Cache, PAGE_TOKENS
from .engine.backend import EngineBackend
from .engine.generate import Finished, GenerationStats, Request, run_requests
from .engine.step import SequenceStep, Stepper
from .loading import build_model, parse_dtype
from .registry import load_config
from .sampling import SamplingParams
from .weights.loader import load_checkpoint

Prompt = Union[Sequence[int], torch.Tensor]


def _as_list(p: Prompt) -> List[int]:
    if isinstance(p, torch.Tensor):
        return [int(x) for x in p.reshape(-1).tolist()]
    return [int(x) for x in p]


class LLM:
    def __init__(self, path: str, memory_limit: float = 0.8, chunk_length: int = 1024, dtype=None,
                 cuda_graph: bool = False, temperature: float = 0.0, random_seed: Optional[int] = None,
                 top_p: float = 1.0, max_batch: int = 64, max_tokens: Optional[int] = None,
                 max_seq_tokens: Optional[int] = None, device: str = "cuda:0", apply_sparse: bool = True,
                 use_arena: bool = True):
        """``apply_sparse`` False runs a model whose configuration has a ``sparse_config`` with dense attention
        (the reference's switch of the same name, cpmcu/llm.py:32, chooses the other way round).  ``use_arena``
        False leaves every tensor to torch's allocator (``max_tokens`` must then be given)."""
        self.use_arena = bool(use_arena)
        self.storage = None
        self.path = path
        self.arch, self.config = load_config(path)
        if not apply_sparse and getattr(self.config, "sparse_config", None) is not None:
            import dataclasses
            self.config = dataclasses.replace(self.config, sparse_config=None)
        self.dtype = parse_dtype(dtype if dtype is not None else getattr(self.config, "torch_dtype", "bfloat16"))
        self.device = device
        self.memory_limit = float(memory_limit)
        self.chunk_length = int(chunk_length)
        self.cuda_graph = bool(cuda_graph)
        self.temperature = float(temperature)
        self.top_p = float(top_p)
        self.seed = 0 if random_seed is None else int(random_seed)
        self.max_batch = int(max_batch)
        self.max_tokens = max_tokens
        self.max_seq_tokens = max_seq_tokens
        self.model = build_model(self.arch, self.config, self.dtype, device)
        self.ops = self.model.ops
        self.tokenizer = None
        self.cache: Optional[Cache] = None
        self.stepper: Optional[Stepper] = None
        self.backend: Optional[EngineBackend] = None
        self.max_total_length = 0
        self.last_stats: Optional[GenerationStats] = None

    # ---- storage ----
    def _weight_bytes(self) -> int:
        es = self.ops.element_size
        total = 0
        for spec in self.model.weight_specs().values():
            n = 1
            for s in spec.shape:
                n *= s
            total += n * (es if spec.role == "matrix" else 4)
        return total

    def init_storage(self) -> int:
        """Lays out the storage (one arena: weights, step workspace, per-sequence state, key-value pages; see
        cpmcu_b200.engine.storage) and returns the number of tokens the longest sequence may hold (the reference
        returns its ``max_total_length`` here, cpmcu/llm.py:115-116).  The cache holds ``max_tokens`` tokens, or
        what ``memory_limit`` leaves.  Raises cpmcu_b200.memory.PoolExhausted (a MemoryError) when something does
        not fit."""
        if self.use_arena:
            from .engine.storage import make_storage
            self.storage = make_storage(self.model, self.chunk_length, self.max_batch, self.max_tokens,
                                        None if self.max_tokens is not None else self.memory_limit, self.max_seq_tokens)
            self.cache = self.storage.cache
        else:
            needs = self.model.cache_needs()
            tokens = self.max_tokens
            if tokens is None:
                raise ValueError("without the arena the cache's size has to be given (max_tokens)")
            tokens = (int(tokens) // PAGE_TOKENS) * PAGE_TOKENS
            per_seq = self.max_seq_tokens or min(tokens, max(self.model.spec.max_positions, 4096) * 8)
            self.cache = Cache(needs, max_tokens=tokens, dtype=self.dtype, device=self.device,
                               n_slots=min(max(2, tokens // PAGE_TOKENS), self.max_batch * 2 + 2), max_seq_tokens=per_seq,
                               max_step_tokens=self.chunk_length)
        self.stepper = Stepper(self.model, self.cache, chunk_tokens=self.chunk_length, graph_prompts=self.cuda_graph)
        self.max_total_length = self.cache.max_pages_per_seq * PAGE_TOKENS
        return self.max_total_length

    def load_from_hf(self) -> None:
        """Loads the folder's safetensors by tensor name (cpmcu/llm.py:177-192)."""
        arch, config = self.arch, self.config
        adapt = (lambda name, t: arch.adapt_tensor(config, name, t)) if arch.adapt_tensor else None
        tensors = load_checkpoint(self.path, self.model.weight_specs(), self.dtype, self.device, adapt,
                                  arch.ignore_tensor)
        self.model.load_weights(tensors)

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Weights that are already on the device, by tensor name (random weights made in place)."""
        self.model.load_weights(tensors)

    def _ready(self) -> EngineBackend:
        if self.stepper is None:
            self.init_storage()
        if not self.model.loaded:
            self.load_from_hf()
        if self.backend is None:
            self.backend = EngineBackend(self.stepper, self.max_batch, self.cuda_graph, self.seed)
        return self.backend

    # ---- generation ----
    def generate_batch(self, prompts: Sequence[Prompt], generation_length: int = 100,
                       terminators: Sequence[int] = (), temperature: Optional[float] = None,
                       top_p: Optional[float] = None,
                       on_token: Optional[Callable[[int, int, bool], None]] = None) -> List[Finished]:
        """Generates for a batch of prompts of unequal lengths; results in the prompts' order."""
        backend = self._ready()
        sp = SamplingParams(self.temperature if temperature is None else float(temperature),
                            self.top_p if top_p is None else float(top_p))
        reqs = [Request(_as_list(p), int(generation_length), sp, tuple(int(t) for t in terminators), key=i)
                for i, p in enumerate(prompts)]
        results, stats = run_requests(backend, reqs, on_token, sync=torch.cuda.synchronize)
        self.last_stats = stats
        return results

    def generate(self, input_ids: Prompt, generation_length: int = 100, terminators: Sequence[int] = (),
                 use_stream: bool = False, progress_callback=None, temperature: Optional[float] = None):
        """One prompt, as the reference's ``generate`` (cpmcu/llm.py:261-376): returns
        ``(tokens, decode_time, prefill_time)``, or with ``use_stream`` a generator of
        dictionaries {'token', 'text', 'is_finished', 'prefill_time', 'decode_time'}."""
        prompt = _as_list(input_ids)
        if progress_callback:
            progress_callback("begin", {"total_tokens": len(prompt)})
        if not use_stream:
            res = self.generate_batch([prompt], generation_length, terminators, temperature)[0]
            if progress_callback:
                progress_callback("finish", {"total_time": self.last_stats.prefill_time})
            return res.tokens, self.last_stats.decode_time, self.last_stats.prefill_time
        return self._stream(prompt, generation_length, terminators, temperature)

    def _stream(self, prompt, generation_length, terminators, temperature) -> Iterator[dict]:
        import queue
        import threading

        q: "queue.Queue" = queue.Queue()
        t_start = time.perf_counter()

        def on_token(_i, token, done):
            q.put((token, done, time.perf_counter() - t_start))

        def work():
            try:
                self.generate_batch([prompt], generation_length, terminators, temperature, on_token=on_token)
            except BaseException as e:  # surfaced in the consumer
                q.put(e)
            q.put(None)

        threading.Thread(target=work, daemon=True).start()
        first = True
        first_time = 0.0
        while True:
            item = q.get()
            if item is None:
                return
            if isinstance(item, BaseException):
                raise item
            token, done, t = item
            text = self.tokenizer.decode([token], skip_special_tokens=True) if self.tokenizer else ""
            if first:
                first_time = t
            yield {"token": token, "text": text, "is_finished": done,
                   "prefill_time": t if first else 0.0, "decode_time": 0.0 if first else t - first_time}
            first = False

    # ---- the step function, for callers that drive it themselves ----
    def step(self, batch: Sequence[SequenceStep]) -> Optional[torch.Tensor]:
        self._ready()
        return self.stepper.step(batch)

    def print_perf_summary(self) -> None:
        s = self.last_stats
        if s is None:
            return
        print(f"prefill: {s.prompt_tokens} tokens in {s.prefill_time:.3f} s "
              f"({s.prompt_tokens / max(s.prefill_time, 1e-9):.1f} tok/s)")
        print(f"decode: {s.generated_tokens} tokens in {s.decode_time:.3f} s "
              f"({s.generated_tokens / max(s.decode_time, 1e-9):.1f} tok/s, {s.decode_steps} steps)")
