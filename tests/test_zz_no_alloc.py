"""The decode attention entry point that brings its own scratch memory
(cpm_decode_attention_bf16_static), called through its exported C symbol.

It is for callers that cannot allocate device memory where they need attention; see
cpmcu_b200/csrc/cpm_no_alloc.h.  The test checks it against the ordinary entry point,
which takes scratch from the caller, on two calls in a row with different batches: the
second call finds the first call's partial results still in the shared array and must
not be disturbed by them.  This file sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2          # the bf16 kernel tolerance of tests/test_gpu_kernels.py
SCRATCH_FLOATS = 4 * 1024 * 1024


def _entry():
    from cpmcu_b200.ops import build
    lib = ctypes.CDLL(build.build())
    fn = lib.cpm_decode_attention_bf16_static
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, ctypes.c_float, P, ctypes.c_char_p, I]
    fn.restype = I
    return fn


def _case(ops, lens, n_heads, n_kv, d, seed):
    """A cache filled with random keys and values for sequences of ``lens``, and one query per sequence."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts.base import CacheNeeds

    cache = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d)], max_tokens=64 * 64, dtype=torch.bfloat16, device="cuda:0")
    slots = cache.open_sequences(len(lens))
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
        cache.set_length(s, n)
    cache.sync()
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    qkv = torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g).bfloat16().cuda()
    positions = torch.cat([torch.arange(n) for n in lens]).int().cuda()
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    sl = torch.tensor(slots, dtype=torch.int32).cuda()
    q = ops.rope_store(qkv, n_heads, n_kv, d, positions, token_seq, sl, lane.page_table, lane.k, lane.v, None, 1.0, 0)
    last = (torch.tensor(lens).cumsum(0) - 1).cuda()
    # the same attention in plain fp32 torch, from the rows that went into the cache (no rotation was applied)
    rows = qkv.float().cpu().view(T, n_heads + 2 * n_kv, d)
    group, want, o = n_heads // n_kv, [], 0
    for n in lens:
        qs, ks, vs = rows[o + n - 1, :n_heads], rows[o:o + n, n_heads:n_heads + n_kv], rows[o:o + n, n_heads + n_kv:]
        heads = [torch.softmax((ks[:, h // group] @ qs[h]) / math.sqrt(d), dim=0) @ vs[:, h // group] for h in range(n_heads)]
        want.append(torch.cat(heads))
        o += n
    _case.reference = torch.stack(want)
    return cache, lane, q[last].contiguous(), torch.tensor(lens, dtype=torch.int32).cuda(), sl


def _call(fn, lane, q, kv_len, sl, n_kv, n_splits, scale):
    n, n_heads, d = q.shape
    out = torch.empty(n, n_heads * d, dtype=torch.bfloat16, device="cuda:0")
    err = ctypes.create_string_buffer(256)
    status = fn(q.data_ptr(), lane.k.data_ptr(), lane.v.data_ptr(), out.data_ptr(), kv_len.data_ptr(), sl.data_ptr(),
                lane.page_table.data_ptr(), lane.page_table.shape[1], n, n_heads, n_kv, d, n_splits, scale,
                torch.cuda.current_stream().cuda_stream, err, 256)
    return status, out, err.value.decode()


def test_static_scratch_entry_matches_the_ordinary_one_twice():
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.bfloat16, "cuda:0")
    fn = _entry()
    # first call: many shares, long sequences; second call: other sizes, fewer shares, shorter sequences,
    # so that most of what the first call left in the array is stale when the second one runs
    for lens, n_heads, n_kv, d, splits, seed in (([700, 64, 333, 1], 32, 2, 128, 16, 1), ([65, 130], 6, 3, 64, 2, 2)):
        cache, lane, q, kv_len, sl = _case(ops, lens, n_heads, n_kv, d, seed)
        scale = 1 / math.sqrt(d)
        want = ops.decode_attention(q, lane.k, lane.v, kv_len, sl, lane.page_table, n_kv, scale, n_splits=splits)
        torch.cuda.synchronize()
        status, got, msg = _call(fn, lane, q, kv_len, sl, n_kv, splits, scale)
        torch.cuda.synchronize()
        assert status == 0, msg
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < TOL, err
        ref = _case.reference                      # not only the two entry points against each other
        assert float((got.float().cpu() - ref).abs().max() / ref.abs().max()) < TOL


def test_static_scratch_entry_refuses_what_does_not_fit():
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.bfloat16, "cuda:0")
    fn = _entry()
    cache, lane, q, kv_len, sl = _case(ops, [10] * 40, 32, 2, 128, 3)
    need = 40 * 2 * 1 * 64 * (16 * 128 + 32)
    assert need > SCRATCH_FLOATS
    status, _, msg = _call(fn, lane, q, kv_len, sl, 2, 64, 0.1)
    assert status == -2 and str(need) in msg and str(SCRATCH_FLOATS) in msg
    status, _, msg = _call(fn, lane, q, kv_len, sl, 2, 4, 0.1)          # the same batch with fewer shares fits
    torch.cuda.synchronize()
    assert status == 0, msg
