"""The generation loop: requests in, token lists out.

Requests are taken in order, as many per batch as the batch limit and the cache
allow; a batch's prompts run in one step (chunked when long), then one token per
sequence per step; a sequence that draws a stop token or reaches its length leaves
the batch and gives its slot and pages back while the others go on; when a batch is
done the next one starts.  The reference's loop handles one prompt
(cpmcu/llm.py:261-376): its ``generation_length`` counts the token that comes out of
the prompt, a stop token is appended before the loop ends, and so it is here.

The loop's decisions are in this file and use a backend with four calls, so they
can be tested without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Protocol, Sequence

from ..cache import CacheFull, pages_for
from ..sampling import SamplingParams


class Backend(Protocol):
    """What the loop needs from an engine."""

    def capacity_pages(self) -> int: ...
    def max_batch(self) -> int: ...

    def prefill(self, prompts: Sequence[Sequence[int]], keys: Sequence[int],
                sampling: Sequence[SamplingParams]) -> List[int]:
        """Opens a sequence per prompt, runs the prompts, returns each one's first token."""

    def decode(self, live: Sequence[int], last_tokens: Sequence[int], keys: Sequence[int],
               steps_done: Sequence[int], sampling: Sequence[SamplingParams], changed: bool) -> List[int]:
        """One token for each live sequence (indices into the batch given to prefill)."""

    def finish(self, index: int) -> None:
        """The sequence at ``index`` of the batch is done; what it holds is given back."""

    def abort(self) -> None:
        """Something failed in the middle of a batch: every sequence of it that is still open is closed."""

    # Optional: ``max_sequence_pages()`` (the most pages one sequence may hold) and ``vocab_size()``; with them
    # a request that cannot run is refused before anything is opened.


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int
    sampling: SamplingParams = SamplingParams()
    stop_token_ids: Sequence[int] = ()
    key: int = 0                       # random key of the request (its index, by default)


@dataclass
class Finished:
    tokens: List[int] = field(default_factory=list)
    reason: str = ""                   # "stop" or "length"


@dataclass
class GenerationStats:
    prefill_time: float = 0.0
    decode_time: float = 0.0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    decode_steps: int = 0
    batches: int = 0


def plan_batches(requests: Sequence[Request], max_batch: int, capacity_pages: int,
                 max_sequence_pages: Optional[int] = None, vocab_size: Optional[int] = None) -> List[List[int]]:
    """Cuts the requests, in order, into batches that fit: at most ``max_batch`` sequences,
    and pages for every sequence grown to its full length.  A request that can never run (longer than
    the cache or than one sequence may be, a token id outside the vocabulary) is refused here, before
    any sequence is opened."""
    batches: List[List[int]] = []
    cur: List[int] = []
    pages = 0
    for i, r in enumerate(requests):
        need = pages_for(len(r.prompt) + max(0, r.max_new_tokens))
        if need > capacity_pages:
            raise CacheFull(f"request {i}: {len(r.prompt)} prompt + {r.max_new_tokens} new tokens need {need} pages, "
                            f"the cache has {capacity_pages}")
        if max_sequence_pages is not None and need > max_sequence_pages:
            raise CacheFull(f"request {i}: {len(r.prompt)} prompt + {r.max_new_tokens} new tokens need {need} pages, "
                            f"one sequence may hold {max_sequence_pages}")
        if vocab_size is not None:
            bad = next((t for t in r.prompt if not 0 <= int(t) < vocab_size), None)
            if bad is not None:
                raise ValueError(f"request {i}: token id {bad} is outside the vocabulary [0, {vocab_size})")
        if cur and (len(cur) >= max_batch or pages + need > capacity_pages):
            batches.append(cur)
            cur, pages = [], 0
        cur.append(i)
        pages += need
    if cur:
        batches.append(cur)
    return batches


def run_requests(backend: Backend, requests: Sequence[Request],
                 on_token: Optional[Callable[[int, int, bool], None]] = None,
                 sync: Optional[Callable[[], None]] = None) -> (List[Finished], GenerationStats):
    """Generates for every request; ``on_token(request index, token, is_last)`` is called as
    tokens appear."""
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise ValueError(f"request {i} has an empty prompt")
    results = [Finished() for _ in requests]
    stats = GenerationStats()
    sync = sync or (lambda: None)
    per_seq = getattr(backend, "max_sequence_pages", None)
    vocab = getattr(backend, "vocab_size", None)
    plan = plan_batches(requests, backend.max_batch(), backend.capacity_pages(),
                        per_seq() if per_seq else None, vocab() if vocab else None)
    try:
        _run_batches(backend, requests, plan, results, stats, on_token, sync)
    except BaseException:
        abort = getattr(backend, "abort", None)
        if abort:
            abort()                      # nothing of a failed batch stays held for the next call
        raise
    return results, stats


def _run_batches(backend, requests, plan, results, stats, on_token, sync) -> None:
    for batch in plan:
        stats.batches += 1
        reqs = [requests[i] for i in batch]
        keys = [r.key for r in reqs]
        sampling = [r.sampling for r in reqs]
        live: List[int] = []
        last: List[int] = [0] * len(batch)
        runnable = [j for j, r in enumerate(reqs) if r.max_new_tokens > 0]
        for j, r in enumerate(reqs):
            if r.max_new_tokens <= 0:
                results[batch[j]].reason = "length"
        if not runnable:
            continue
        sync()
        t0 = time.perf_counter()
        first = backend.prefill([reqs[j].prompt for j in runnable], [keys[j] for j in runnable],
                                [sampling[j] for j in runnable])
        sync()
        stats.prefill_time += time.perf_counter() - t0
        stats.prompt_tokens += sum(len(reqs[j].prompt) for j in runnable)

        def take(j: int, pos: int, token: int) -> bool:
            """Records a token; True if the sequence goes on."""
            res, r = results[batch[j]], reqs[j]
            res.tokens.append(token)
            stats.generated_tokens += 1
            done = token in r.stop_token_ids or len(res.tokens) >= r.max_new_tokens
            if done:
                res.reason = "stop" if token in r.stop_token_ids else "length"
                backend.finish(pos)
            if on_token:
                on_token(batch[j], token, done)
            return not done

        # positions in the backend's batch are indices into ``runnable``
        for pos, j in enumerate(runnable):
            if take(j, pos, first[pos]):
                live.append(pos)
                last[pos] = first[pos]
        changed = True
        t0 = time.perf_counter()
        while live:
            toks = backend.decode(live, [last[p] for p in live], [keys[runnable[p]] for p in live],
                                  [len(results[batch[runnable[p]]].tokens) for p in live],
                                  [sampling[runnable[p]] for p in live], changed)
            stats.decode_steps += 1
            still: List[int] = []
            for p, tok in zip(live, toks):
                if take(runnable[p], p, tok):
                    still.append(p)
                    last[p] = tok
            changed = len(still) != len(live)
            live = still
        sync()
        stats.decode_time += time.perf_counter() - t0
