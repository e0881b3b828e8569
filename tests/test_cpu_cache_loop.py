"""The cache's bookkeeping (no slot or page lost, held twice or freed twice), the chunk
planner and the generation loop's decisions, without a device."""
import random

import pytest
import torch

from cpmcu_b200.cache import Cache, CacheFull, FreeList, HandleError, pages_for
from cpmcu_b200.engine.generate import Request, plan_batches, run_requests
from cpmcu_b200.engine.step import plan_chunks
from cpmcu_b200.parts.base import CacheNeeds
from cpmcu_b200.sampling import SamplingParams


def test_free_list():
    f = FreeList(4, "page")
    a = f.take(3)
    assert a == [0, 1, 2] and f.n_free == 1
    with pytest.raises(CacheFull):
        f.take(2)
    f.give_back([1])
    with pytest.raises(HandleError):
        f.give_back([1])                    # freed twice
    with pytest.raises(HandleError):
        f.give_back([3])                    # never handed out
    assert f.take(2) == [1, 3]              # lowest first


def _cache(n_tokens=64 * 10, **kw):
    needs = [CacheNeeds(kv_heads=2, head_dim=16)] * 2 + [CacheNeeds(kv_heads=1, head_dim=32, window=64)] + \
            [CacheNeeds(state={"acc": ((8,), torch.float32)})]
    return Cache(needs, max_tokens=n_tokens, dtype=torch.float32, device="cpu", **kw)


def test_groups_have_their_own_storage():
    c = _cache()
    assert len(c.groups) == 3
    g0 = c.lane(0).group
    assert c.lane(1).group is g0 and c.lane(2).group is not g0
    assert c.lane(0).k.shape == (10, 2, 64, 16) and c.lane(2).k.shape == (10, 1, 64, 32)
    assert c.lane(0).v.shape == (10, 2, 16, 64)
    assert c.lane(3).k is None and c.lane(3).state["acc"].shape == (c.n_slots, 8)
    assert c.lane(0).k.data_ptr() != c.lane(1).k.data_ptr()


def test_random_open_grow_close_never_loses_a_page():
    rng = random.Random(0)
    c = _cache(64 * 20, n_slots=6)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and c.slots.n_free:
            s = c.open_sequence()
            assert s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            new = live[s] + rng.randint(1, 150)
            try:
                c.reserve(s, new)
                c.set_length(s, new)
                live[s] = new
            except CacheFull:
                pass                                         # all or nothing: nothing was taken
        elif live:
            s = rng.choice(list(live))
            c.close_sequence(s)
            del live[s]
            with pytest.raises(HandleError):
                c.close_sequence(s)                          # closed twice
        c.check_consistent()
        for g in c.groups:
            if g.needs.window:
                # pages whose keys are all before the window of any later query have gone back
                want = sum(pages_for(n) - max(0, n - g.needs.window + 1) // 64 for n in live.values())
            else:
                want = sum(pages_for(n) for n in live.values())
            assert g.pages.n_held == want
    for s in list(live):
        c.close_sequence(s)
    assert c.tokens_held() == 0 and c.slots.n_free == 6


def test_state_is_cleared_when_a_slot_is_reused():
    c = _cache()
    s = c.open_sequence()
    c.lane(3).state["acc"][s] += 5
    c.close_sequence(s)
    s2 = c.open_sequence()
    assert s2 == s and float(c.lane(3).state["acc"][s2].abs().sum()) == 0


def test_page_table_follows_the_pages():
    c = _cache()
    a, b = c.open_sequences(2)
    c.reserve(a, 70); c.reserve(b, 10); c.reserve(a, 200)
    c.sync()
    g = c.groups[0]
    assert g.page_table[a, :4].tolist() == g.pages_of_slot[a] == [0, 1, 3, 4]
    assert g.page_table[b, :1].tolist() == [2]
    with pytest.raises(CacheFull, match="pages"):
        c.reserve(b, 64 * 10)


def test_plan_chunks():
    chunks = plan_chunks([5, 17, 33], 16)
    assert [(c.begin, c.end) for c in chunks] == [(0, 16), (16, 32), (32, 48), (48, 55)]
    assert chunks[0].pieces == [(0, 0, 5), (1, 0, 11)] and chunks[1].pieces == [(1, 11, 6), (2, 0, 10)]
    covered = [0] * 3
    for c in chunks:
        assert sum(n for _, _, n in c.pieces) == c.end - c.begin <= 16
        for i, first, n in c.pieces:
            assert first == covered[i]
            covered[i] += n
    assert covered == [5, 17, 33]
    assert len(plan_chunks([3, 4], 100)) == 1


class FakeBackend:
    """Scripted tokens: sequence with key k produces k*100 + n as its n-th token."""

    def __init__(self, pages=100, batch=3):
        self.pages, self.batch = pages, batch
        self.open, self.log, self.n_open_max = {}, [], 0

    def capacity_pages(self): return self.pages
    def max_batch(self): return self.batch

    def prefill(self, prompts, keys, sampling):
        assert not self.open, "a batch started before the last one ended"
        self.open = {i: k for i, k in enumerate(keys)}
        self.n_open_max = max(self.n_open_max, len(self.open))
        self.log.append(("prefill", [len(p) for p in prompts]))
        return [k * 100 for k in keys]

    def decode(self, live, last_tokens, keys, steps_done, sampling, changed):
        assert all(i in self.open for i in live)
        assert [self.open[i] for i in live] == list(keys)
        assert last_tokens == [k * 100 + n - 1 for k, n in zip(keys, steps_done)]
        self.log.append(("decode", list(live), changed))
        return [k * 100 + n for k, n in zip(keys, steps_done)]

    def finish(self, index):
        del self.open[index]                 # KeyError if finished twice


def test_loop_batches_stops_and_early_leavers():
    reqs = [Request([1] * 5, 4, key=0), Request([1] * 9, 8, stop_token_ids=(102,), key=1),
            Request([1] * 2, 1, key=2), Request([1] * 70, 3, key=3), Request([1] * 3, 0, key=4)]
    be = FakeBackend(batch=3)
    res, stats = run_requests(be, reqs)
    assert [r.tokens for r in res] == [[0, 1, 2, 3], [100, 101, 102], [200], [300, 301, 302], []]
    assert [r.reason for r in res] == ["length", "stop", "length", "length", "length"]
    assert not be.open and stats.batches == 2 and stats.generated_tokens == 11
    # batch 1: request 2 leaves after the prompt, request 1 after its stop token, request 0 last
    assert be.log[0] == ("prefill", [5, 9, 2])
    assert be.log[1] == ("decode", [0, 1], True) and be.log[2] == ("decode", [0, 1], False)
    assert be.log[3] == ("decode", [0], True)
    assert be.log[4] == ("prefill", [70])


def test_loop_respects_cache_capacity():
    reqs = [Request([1] * 100, 28, key=i) for i in range(5)]         # two pages each
    assert plan_batches(reqs, max_batch=8, capacity_pages=5) == [[0, 1], [2, 3], [4]]
    with pytest.raises(CacheFull):
        plan_batches([Request([1] * 1000, 10)], 8, 5)
    with pytest.raises(ValueError):
        run_requests(FakeBackend(), [Request([], 3)])


def test_sampling_params():
    assert SamplingParams().greedy and not SamplingParams(0.7).greedy
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0)


def test_window_group_gives_pages_back_as_the_window_moves():
    needs = [CacheNeeds(kv_heads=1, head_dim=16), CacheNeeds(kv_heads=1, head_dim=16, window=100)]
    c = Cache(needs, max_tokens=64 * 64, dtype=torch.float32, device="cpu", n_slots=3, max_step_tokens=130)
    full, win = c.lane(0).group, c.lane(1).group
    assert win.n_pages == 3 * (pages_for(100 + 130) + 1) and full.n_pages == 64      # sized by window + step
    s = c.open_sequence()
    length = 0
    for step in [130, 130, 1, 1, 64, 1] + [1] * 200 + [130] * 5:
        c.reserve(s, length + step)
        length += step
        c.set_length(s, length)
        c.check_consistent()
        assert full.pages_held(s) == pages_for(length)
        first_needed = max(0, length - 100 + 1) // 64
        assert win.pages_held(s) == pages_for(length) - first_needed
        assert win.pages_held(s) <= pages_for(100) + 1
        # the pages of the keys that later queries see are all there
        assert all(p >= 0 for p in win.pages_of_slot[s][first_needed:])
    c.close_sequence(s)
    assert win.pages.n_held == 0 and full.pages.n_held == 0
    c.check_consistent()


class FailingBackend(FakeBackend):
    """Holds slots like an engine does; its n-th call of ``fail_at`` raises."""

    def __init__(self, fail_at, **kw):
        super().__init__(**kw)
        self.fail_at, self.aborted = fail_at, 0

    def max_sequence_pages(self): return 4
    def vocab_size(self): return 50

    def prefill(self, prompts, keys, sampling):
        out = super().prefill(prompts, keys, sampling)
        if self.fail_at == "prefill":
            raise RuntimeError("a step failed")
        return out

    def decode(self, live, last_tokens, keys, steps_done, sampling, changed):
        if self.fail_at == "decode":
            raise RuntimeError("a step failed")
        return super().decode(live, last_tokens, keys, steps_done, sampling, changed)

    def abort(self):
        self.aborted += 1
        self.open = {}


def test_a_failing_request_leaves_nothing_held():
    good = [Request([1] * 5, 4, key=0), Request([1] * 9, 3, key=1)]
    for where in ("prefill", "decode"):
        be = FailingBackend(where)
        with pytest.raises(RuntimeError, match="a step failed"):
            run_requests(be, good)
        assert be.aborted == 1 and not be.open
    # requests that can never run are refused before any sequence is opened
    be = FailingBackend(None)
    with pytest.raises(CacheFull, match="one sequence may hold 4"):
        run_requests(be, good + [Request([1] * 300, 10, key=2)])
    with pytest.raises(ValueError, match="token id 50 is outside"):
        run_requests(be, good + [Request([1, 50], 10, key=2)])
    assert be.log == [] and not be.open
    res, _ = run_requests(be, good)                                 # and the backend is still usable
    assert [r.tokens for r in res] == [[0, 1, 2, 3], [100, 101, 102]]


def test_engine_backend_gives_slots_back_when_a_step_fails():
    """The device backend over a stand-in stepper: a prompt's step raises; the slots opened for the batch, and the
    pages reserved for its earlier sequences, are all given back."""
    from cpmcu_b200.engine.backend import EngineBackend

    cache = Cache([CacheNeeds(kv_heads=1, head_dim=16)], max_tokens=64 * 8, dtype=torch.float32, device="cpu", n_slots=6,
                  max_seq_tokens=64 * 3)

    class Ops:
        device = "cpu"
        def raise_on_kernel_error(self): pass

    class StandInStepper:
        ops, vocab_size = Ops(), 50
        def __init__(self): self.cache = cache
        def open(self, n): return cache.open_sequences(n)
        def close(self, s): cache.close_sequence(s)
        def step(self, batch):
            for b in batch:
                cache.reserve(b.slot, len(b.tokens))        # the second sequence is too long for one sequence
            return None

    be = EngineBackend.__new__(EngineBackend)
    be.stepper, be.ops, be.seed, be._max_batch = StandInStepper(), Ops(), 0, 4
    be.slots, be.open, be.h2d_bytes, be.d2h_bytes = [], set(), 0, 0
    with pytest.raises(CacheFull, match="pages"):
        be.prefill([[1] * 70, [1] * 400, [1] * 5], [0, 1, 2], [SamplingParams()] * 3)
    cache.check_consistent()
    assert cache.slots.n_held == 0 and cache.tokens_held() == 0
    assert be.max_sequence_pages() == 3 and be.vocab_size() == 50


def test_decode_steps_take_pages_only_at_page_edges():
    c = _cache(64 * 12, n_slots=4)
    a, b = c.open_sequence(), c.open_sequence()
    c.reserve(a, 63); c.set_length(a, 63)
    c.reserve(b, 64); c.set_length(b, 64)
    assert c.grow_by_one([a, b]) is True           # b's last page is full
    c.grown_by_one([a, b])
    assert (c.length(a), c.length(b)) == (64, 65)
    assert c.grow_by_one([b]) is False             # room left in b's second page
    assert c.grow_by_one([a, b]) is True           # now a's page is full
    c.grown_by_one([a, b])
    c.check_consistent()
    for g in c.groups:
        if not g.needs.window:
            assert g.pages_held(a) == 2 and g.pages_held(b) == 2
    # all or nothing: a step that cannot get its pages takes none
    small = Cache([CacheNeeds(kv_heads=1, head_dim=16)], max_tokens=64 * 3, dtype=torch.float32, device="cpu", n_slots=3)
    x, y = small.open_sequence(), small.open_sequence()
    small.reserve(x, 64); small.set_length(x, 64)
    small.reserve(y, 128); small.set_length(y, 128)
    with pytest.raises(CacheFull):
        small.grow_by_one([x, y])
    assert small.groups[0].pages.n_held == 3
    small.check_consistent()
