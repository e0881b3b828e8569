"""The generation loop's backend on the device: prompts through the step function,
decode steps through the decode runner, sampling by the library's kernel."""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..sampling import SamplingParams
from .decode import DecodeRunner
from .step import SequenceStep, Stepper


class EngineBackend:
    def __init__(self, stepper: Stepper, max_batch: int = 64, use_graph: bool = True, seed: int = 0):
        self.stepper = stepper
        self.ops = stepper.ops
        self.seed = int(seed)
        self.runner = DecodeRunner(stepper, use_graph=use_graph, seed=seed)
        self._max_batch = int(max_batch)
        self.slots: List[int] = []
        self.open: set = set()              # slots of the current batch that are not finished yet
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def capacity_pages(self) -> int:
        return self.stepper.cache.n_pages - 1          # one page belongs to the decode runner's padding

    def max_batch(self) -> int:
        return min(self._max_batch, self.stepper.cache.n_slots - 1)

    def _sample(self, logits: torch.Tensor, keys: Sequence[int], steps: Sequence[int],
                sampling: Sequence[SamplingParams]) -> List[int]:
        n = len(keys)
        if all(p.greedy for p in sampling):
            out = self.ops.sample(logits)
        else:
            i = torch.tensor(list(keys) + list(steps), dtype=torch.int32).view(2, n).to(self.ops.device)
            f = torch.tensor([p.temperature for p in sampling] + [p.top_p for p in sampling],
                             dtype=torch.float32).view(2, n).to(self.ops.device)
            out = self.ops.sample(logits, f[0].contiguous(), f[1].contiguous(), self.seed, i[0].contiguous(),
                                  i[1].contiguous())
        self.d2h_bytes += 4 * n
        return out.cpu().tolist()

    def max_sequence_pages(self) -> int:
        return self.stepper.cache.max_pages_per_seq

    def vocab_size(self) -> int:
        return self.stepper.vocab_size

    def prefill(self, prompts, keys, sampling) -> List[int]:
        self.slots = self.stepper.open(len(prompts))
        self.open = set(self.slots)
        try:
            batch = [SequenceStep(s, list(p), [len(p) - 1]) for s, p in zip(self.slots, prompts)]
            self.h2d_bytes += 4 * sum(len(p) for p in prompts)
            logits = self.stepper.step(batch)
            tokens = self._sample(logits, keys, [0] * len(prompts), sampling)
            self.ops.raise_on_kernel_error()            # the host has just waited for the tokens anyway
        except BaseException:
            self.abort()
            raise
        return tokens

    def abort(self) -> None:
        """Closes every sequence of the current batch that is still open (a step failed)."""
        for s in sorted(self.open):
            self.stepper.close(s)
        self.open = set()

    def decode(self, live, last_tokens, keys, steps_done, sampling, changed) -> List[int]:
        if changed:
            self.runner.start([self.slots[p] for p in live], last_tokens, keys, steps_done, sampling)
            self.h2d_bytes += 4 * 7 * len(live)
        else:
            self.runner.feed(last_tokens)               # the step's inputs: host tokens, pinned, every step
            self.h2d_bytes += 4 * len(live)
        self.runner.step()
        self.d2h_bytes += 4 * len(live)
        return self.runner.read_tokens()

    def finish(self, index: int) -> None:
        self.stepper.close(self.slots[index])
        self.open.discard(self.slots[index])
