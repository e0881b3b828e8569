"""The arena and its regions, the workspace's lifetimes, the sizing of the storage and its errors, without a device."""
import pytest
import torch

from cpmcu_b200.cache import Cache, CacheFull
from cpmcu_b200.memory import ALIGN, Arena, PoolExhausted, Workspace, plan_storage
from cpmcu_b200.parts.base import CacheNeeds
from tests import configs


def test_regions_are_carved_in_order_and_name_themselves_when_full():
    arena = Arena(64 * 1024, "cpu")
    w = arena.carve("weights", 10_000)
    c = arena.carve("cache", 40_000)
    assert w.offset == 0 and c.offset == w.size and w.size % ALIGN == 0
    a = w.tensor((100,), torch.float32)
    b = w.tensor((3, 5), torch.bfloat16, zero=True)
    assert a.data_ptr() % ALIGN == 0 and b.data_ptr() % ALIGN == 0 and b.data_ptr() >= a.data_ptr() + 400
    assert float(b.float().abs().sum()) == 0.0
    a.fill_(7.0)
    assert arena.buffer[:400].view(torch.float32).tolist() == [7.0] * 100            # a view of the one allocation
    with pytest.raises(PoolExhausted, match="region 'weights'") as e:
        w.tensor((10_000,), torch.float32, what="a tensor too many")
    assert e.value.region == "weights" and "a tensor too many" in str(e.value)
    with pytest.raises(PoolExhausted, match="region 'arena'"):
        arena.carve("more", 30_000)
    assert arena.report()["weights"][1] == w.peak


def test_workspace_frames_alternate_and_the_step_is_checked_before_it_runs():
    arena = Arena(1 << 20, "cpu")
    ws = Workspace(arena.carve("workspace", 4096), [arena.carve("frame0", 8192), arena.carve("frame1", 8192)],
                   sized_tokens=64, sized_seqs=4)
    ws.begin_step()
    x = ws.alloc((16,), torch.float32)                       # persistent: lives through the step
    ws.begin_layer(0)
    f0 = ws.alloc((100,), torch.float32)
    f0.fill_(1.0)
    ws.begin_layer(1)
    f1 = ws.alloc((100,), torch.float32)
    f1.fill_(2.0)
    assert float(f0.sum()) == 100.0                          # layer 0's output is intact while layer 1 runs
    ws.begin_layer(2)
    g0 = ws.alloc((100,), torch.float32)
    assert g0.data_ptr() == f0.data_ptr() and float(f1.sum()) == 200.0      # layer 2 takes layer 0's place, not layer 1's
    ws.end_layers()
    y = ws.alloc((16,), torch.float32)
    assert y.data_ptr() > x.data_ptr()
    with pytest.raises(PoolExhausted, match="region 'frame1'"):
        ws.begin_layer(3)
        ws.alloc((4096,), torch.float32)
    ws.require(64, 4)
    with pytest.raises(PoolExhausted, match="128 tokens.*sized for 64"):
        ws.require(128, 1)                                   # a chunk larger than the workspace was sized for
    with pytest.raises(PoolExhausted, match="sequences"):
        ws.require(8, 8)
    assert ws.peaks()[1] >= 400


def test_plan_storage_says_what_does_not_fit():
    def cache_bytes(tokens):                                 # 1 KiB per token and a table that grows with it
        return tokens * 1024 + tokens // 64 * 4 * 10

    tokens, total = plan_storage(10 << 20, 2 << 20, 1 << 20, cache_bytes, None)
    assert tokens % 64 == 0 and cache_bytes(tokens) <= (10 << 20) - (3 << 20) and cache_bytes(tokens + 128) > (7 << 20) - 64 * ALIGN - 200_000
    tokens, total = plan_storage(None, 2 << 20, 1 << 20, cache_bytes, 1000)
    assert tokens == 960 and total >= (3 << 20) + cache_bytes(960)
    with pytest.raises(PoolExhausted, match="region 'cache'.*two pages"):            # memory_limit too small for any cache
        plan_storage((3 << 20) + 64 * ALIGN + 50_000, 2 << 20, 1 << 20, cache_bytes, None)
    with pytest.raises(PoolExhausted, match="region 'weights'"):
        plan_storage(1 << 20, 2 << 20, 1 << 20, cache_bytes, None)
    with pytest.raises(PoolExhausted, match="region 'workspace'"):
        plan_storage(5 << 19, 2 << 20, 1 << 20, cache_bytes, None)
    with pytest.raises(PoolExhausted, match="do not fit the memory limit"):
        plan_storage(4 << 20, 2 << 20, 1 << 20, cache_bytes, 4096)


def test_workspace_is_measured_by_the_models_own_forward_pass():
    from cpmcu_b200.ops.dry import measure_workspace
    from cpmcu_b200.registry import architecture

    arch = architecture("MiniCPMForCausalLM")
    sizes = {}
    for name, cfgd in (("a", configs.tiny_a()), ("b", configs.tiny_b())):
        spec = arch.model_spec(arch.config_class.from_dict(cfgd))
        for chunk in (64, 256):
            p, f, notes = measure_workspace(spec, torch.bfloat16, chunk, 4, 1024)
            assert notes == [] and p > 0 and f > 0
            sizes[(name, chunk)] = (p, f)
        # four times the tokens: up to four times the frame (per-token tensors, plus padding and scratch that do not grow)
        if name == "a":
            assert 2.0 < sizes[(name, 256)][1] / sizes[(name, 64)][1] < 4.5
        else:       # the sparse model's largest tensor is the block selection's scratch for steps of few tokens
            assert sizes[(name, 256)][1] >= sizes[(name, 64)][1]
    p32, f32, _ = measure_workspace(arch.model_spec(arch.config_class.from_dict(configs.tiny_a())), torch.float32, 64, 4, 1024)
    assert f32 > sizes[("a", 64)][1]
    # a frame holds at least the widest tensor of a layer: the gate_up product of 64 tokens
    assert sizes[("a", 64)][1] >= 64 * 176 * 2


def test_cache_inside_regions():
    needs = [CacheNeeds(kv_heads=2, head_dim=16), CacheNeeds(kv_heads=1, head_dim=32, state={"s": ((8,), torch.float32)})]
    counting = Arena(None, None)
    st, pg = counting.carve("state", None), counting.carve("cache", None)
    Cache(needs, max_tokens=64 * 8, dtype=torch.float32, device="meta", n_slots=4, state_region=st, page_region=pg)
    assert pg.peak >= 8 * 64 * (2 * 2 * 16 + 2 * 32) * 4 and st.peak >= 2 * 4 * 8 * 4
    arena = Arena(st.peak + pg.peak + 64 * ALIGN, "cpu")
    c = Cache(needs, max_tokens=64 * 8, dtype=torch.float32, device="cpu", n_slots=4,
              state_region=arena.carve("state", st.peak + 16 * ALIGN), page_region=arena.carve("cache", pg.peak + 16 * ALIGN))
    lo, hi = arena.buffer.data_ptr(), arena.buffer.data_ptr() + arena.total
    for lane in c.lanes:
        for t in (lane.k, lane.v, lane.page_table, *lane.state.values()):
            assert lo <= t.data_ptr() < hi
    s = c.open_sequence()
    c.reserve(s, 200)
    c.set_length(s, 200)
    c.check_consistent()
    with pytest.raises(CacheFull):
        c.reserve(s, 64 * 9)
    small = Arena(1 << 20, "cpu")
    with pytest.raises(PoolExhausted, match="region 'cache'.*key-value pages"):
        Cache(needs, max_tokens=64 * 64, dtype=torch.float32, device="cpu", n_slots=4,
              state_region=small.carve("state", 1 << 16), page_region=small.carve("cache", 1 << 18))


def test_guard_words_show_which_region_was_overrun():
    arena = Arena(64 * 1024, "cpu", guards=True)
    a = arena.carve("frame0", 1024)
    b = arena.carve("frame1", 1024)
    assert b.offset == a.offset + a.size + ALIGN            # a guard lies between them
    t = a.tensor((256,), torch.float32)
    t.fill_(1.0)
    arena.check_guards()
    arena.buffer[a.offset + a.size + 3] = 0                 # one byte past frame0's end
    with pytest.raises(RuntimeError, match="behind region 'frame0'.*byte 3"):
        arena.check_guards()
