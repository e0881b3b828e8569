"""Each kernel alone against a plain PyTorch fp32 reference of the same operation, at
sizes other than the models' (odd widths, group sizes 1/3/8, head sizes 16..256)."""
import math

import pytest
import torch

from tests.plain import minicpm4_plain as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative to the largest reference value; bf16 = one rounding of the output (2^-9) plus input rounding
KTOL = {"float32": 1e-5, "bfloat16": 1e-2}


def _ops(dtype):
    from cpmcu_b200.ops.ops import Ops
    return Ops(DT[dtype], "cuda:0")


def _err(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [24, 72, 1000, 4096])
def test_embed(dtype, hidden):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(1)
    table = torch.randn(333, hidden, generator=g).to(DT[dtype])
    ids = torch.randint(0, 333, (17,), generator=g, dtype=torch.int32)
    got = ops.embed(ids.cuda(), table.cuda(), 12.5)
    want = table.float()[ids.long()] * 12.5
    assert got.dtype == torch.float32
    assert _err(got, want) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [24, 72, 1000, 4096, 13000])
def test_add_rmsnorm(dtype, hidden):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(9, hidden, generator=g) * 3
    delta = torch.randn(9, hidden, generator=g).to(DT[dtype])
    w32 = 1 + 0.1 * torch.randn(hidden, generator=g)
    for w in ([w32] if dtype == "float32" else [w32, w32.to(torch.bfloat16)]):
        xd = x.clone().cuda()
        y = ops.add_rmsnorm(xd, delta.cuda(), 0.37, w.cuda(), 1e-5)
        xs = x + 0.37 * delta.float()
        assert _err(xd, xs) < 1e-6
        want = plain.rms_norm(xs, w.float(), 1e-5)
        assert _err(y, want) < KTOL[dtype]
        # rows mode: compact output, the stream stays as it is
        rows = torch.tensor([7, 0, 3], dtype=torch.int32).cuda()
        xd2 = x.clone().cuda()
        y2 = ops.add_rmsnorm(xd2, delta.cuda(), 0.37, w.cuda(), 1e-5, rows)
        assert torch.equal(xd2.cpu(), x)
        assert _err(y2, want[rows.cpu().long()]) < KTOL[dtype]
        # no addend
        y3 = ops.add_rmsnorm(x.clone().cuda(), None, 0.0, w.cuda(), 1e-5)
        assert _err(y3, plain.rms_norm(x, w.float(), 1e-5)) < KTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_add_and_silu_mul(dtype):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 100, generator=g)
    d = torch.randn(5, 100, generator=g).to(DT[dtype])
    xd = x.clone().cuda()
    ops.residual_add(xd, d.cuda(), -0.5)
    assert _err(xd, x - 0.5 * d.float()) < 1e-6
    gu = (torch.randn(7, 2 * 333, generator=g) * 3).to(DT[dtype])
    got = ops.silu_mul(gu.cuda())
    gate, up = gu.float()[:, :333], gu.float()[:, 333:]
    want = gate * (1 / (1 + torch.exp(-gate))) * up
    assert _err(got, want) < KTOL[dtype]


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 5, 7), (64, 64, 16), (65, 130, 33), (150, 1000, 72), (8, 777, 320)])
def test_gemm_f32(M, N, K):
    ops = _ops("float32")
    g = torch.Generator().manual_seed(4)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    got = ops.linear(a.cuda(), w.cuda(), alpha=0.25)
    want = (a.double() @ w.double().T * 0.25).float()
    assert _err(got, want) < 1e-5
    # a row's result does not depend on the other rows of the batch
    one = ops.linear(a[:1].contiguous().cuda(), w.cuda(), alpha=0.25)
    assert torch.equal(one[0], got[0])


def test_linear_bf16():
    ops = _ops("bfloat16")
    g = torch.Generator().manual_seed(5)
    a, w = torch.randn(37, 72, generator=g).bfloat16(), torch.randn(777, 72, generator=g).bfloat16()
    want = a.float() @ w.float().T
    assert _err(ops.linear(a.cuda(), w.cuda()), want) < KTOL["bfloat16"]
    lg = ops.linear(a.cuda(), w.cuda(), alpha=0.5, out_f32=True)
    assert lg.dtype == torch.float32
    assert _err(lg, want * 0.5) < 1e-5


def _paged_setup(ops, lens, n_kv, d, seed, dtype):
    """Random rotated q/k/v for sequences of ``lens``, stored through rope_store into
    pages handed out in a scrambled order."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts.base import CacheNeeds

    cache = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d)], max_tokens=max(64 * 40, sum(lens) + 64 * 12), dtype=DT[dtype],
                  device="cuda:0")
    # scramble the page order so that logical and physical pages differ
    junk = cache.open_sequences(3)
    for j, s in enumerate(junk):
        cache.reserve(s, 64 * (j + 1))
    slots = cache.open_sequences(len(lens))
    cache.close_sequence(junk[1])
    for s, n in zip(slots, lens):
        cache.reserve(s, n)
        cache.set_length(s, n)
    cache.sync()
    return cache, slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv,d,rot", [(4, 2, 16, 16), (3, 3, 48, 48), (8, 1, 64, 32), (6, 2, 128, 128),
                                                (2, 1, 256, 256), (5, 5, 32, 0)])
def test_rope_store_and_attention(dtype, n_heads, n_kv, d, rot):
    ops = _ops(dtype)
    lens = [1, 70, 200, 64]
    cache, slots = _paged_setup(ops, lens, n_kv, d, 0, dtype)
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(6)
    T = sum(lens)
    qkv = torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g).to(DT[dtype])
    positions = torch.cat([torch.arange(n) for n in lens]).int()
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int()
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / max(rot, 1)))) if rot else None
    mag = 1.3
    q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions.cuda(), token_seq.cuda(),
                       torch.tensor(slots, dtype=torch.int32).cuda(), lane.page_table, lane.k, lane.v,
                       inv_freq.cuda() if rot else None, mag, rot)
    rows = qkv.float().view(T, n_heads + 2 * n_kv, d)
    q_ref, k_ref, v_ref = rows[:, :n_heads], rows[:, n_heads:n_heads + n_kv], rows[:, n_heads + n_kv:]
    if rot:
        def rot_part(u):
            return torch.cat([plain.rotate(u[..., :rot], positions, inv_freq, mag), u[..., rot:]], dim=-1)
        q_ref, k_ref = rot_part(q_ref), rot_part(k_ref)
    assert _err(q, q_ref) < KTOL[dtype]
    # read the cache back through the page table
    table = lane.page_table.cpu()
    o = 0
    for s, n in zip(slots, lens):
        for j in (0, n // 2, n - 1):
            page = int(table[s, j // 64])
            got_k = lane.k[page, :, j % 64].float().cpu()
            got_v = lane.v[page, :, :, j % 64].float().cpu()
            assert _err(got_k, k_ref[o + j]) < KTOL[dtype]
            assert _err(got_v, v_ref[o + j]) < KTOL[dtype]
        o += n
    # attention of all tokens over their sequences
    scale = 1 / math.sqrt(d)
    out = ops.attention_generic(q, lane.k, lane.v, positions.cuda(), token_seq.cuda(),
                                torch.tensor(slots, dtype=torch.int32).cuda(), lane.page_table, n_kv, scale)
    qr = q.float().cpu() if dtype == "bfloat16" else q_ref
    o = 0
    for n in lens:
        kk = k_ref[o:o + n].to(DT[dtype]).float()
        vv = v_ref[o:o + n].to(DT[dtype]).float()
        want = plain.dense_attention(qr[o:o + n], kk, vv, scale).reshape(n, -1)
        assert _err(out[o:o + n], want) < KTOL[dtype], (n,)
        o += n
    # window
    outw = ops.attention_generic(q, lane.k, lane.v, positions.cuda(), token_seq.cuda(),
                                 torch.tensor(slots, dtype=torch.int32).cuda(), lane.page_table, n_kv, scale, window=37)
    o = sum(lens[:2])
    want = plain.dense_attention(qr[o:o + 200], k_ref[o:o + 200].to(DT[dtype]).float(),
                                 v_ref[o:o + 200].to(DT[dtype]).float(), scale, window=37).reshape(200, -1)
    assert _err(outw[o:o + 200], want) < KTOL[dtype]


def test_attention_far_key_stands_out():
    """One key far back is made to dominate: its value must come through whatever page it is in."""
    ops = _ops("float32")
    n_heads, n_kv, d, n = 2, 1, 32, 700
    cache, slots = _paged_setup(ops, [n], n_kv, d, 0, "float32")
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(n, (n_heads + 2) * d, generator=g) * 0.1
    rows = qkv.view(n, n_heads + 2, d)
    far = 130
    rows[far, n_heads] = 4.0                      # key
    rows[n - 1, :n_heads] = 4.0                   # last query matches it
    positions = torch.arange(n).int().cuda()
    token_seq = torch.zeros(n, dtype=torch.int32).cuda()
    sl = torch.tensor(slots, dtype=torch.int32).cuda()
    q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions, token_seq, sl, lane.page_table, lane.k, lane.v,
                       None, 1.0, 0)
    out = ops.attention_generic(q, lane.k, lane.v, positions, token_seq, sl, lane.page_table, n_kv, 1 / math.sqrt(d))
    v_far = rows[far, n_heads + 1]
    assert _err(out[n - 1].view(n_heads, d)[0], v_far) < 1e-3


@pytest.mark.parametrize("vocab", [5, 777, 73448])
def test_sampling(vocab):
    ops = _ops("float32")
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(6, vocab, generator=g) * 3
    logits[1, vocab - 1] = logits[1, 3] = 50.0         # a tie: the lower index wins
    got = ops.sample(logits.cuda()).cpu()
    for r in range(6):
        assert int(got[r]) == plain.sample_token(logits[r], 0.0, 0.0)
    assert int(got[1]) == 3
    temps = torch.tensor([0.8, 0.0, 1.5, 0.3, 1.0, 2.0])
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 0.05, 1.0])
    seq_key = torch.arange(6, dtype=torch.int32)
    for step in range(20):
        step_key = torch.full((6,), step, dtype=torch.int32)
        got = ops.sample(logits.cuda(), temps.cuda(), top_p.cuda(), 1234, seq_key.cuda(), step_key.cuda()).cpu()
        for r in range(6):
            tok = int(got[r])
            if temps[r] == 0:
                assert tok == plain.sample_token(logits[r], 0.0, 0.0)
                continue
            u = plain.philox_uniform(1234, r, step)
            w = plain.sampling_weights(logits[r], float(temps[r]), float(top_p[r]))
            assert w[tok] > 0, "a token outside the nucleus was drawn"
            c = torch.cumsum(w, 0)
            target = u * float(c[-1])
            slack = 1e-5 * float(c[-1])
            lo = float(c[tok - 1]) if tok > 0 else 0.0
            assert lo - slack <= target <= float(c[tok]) + slack, (r, step, tok, lo, target, float(c[tok]))


@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 1, 32), (6, 2, 64), (16, 16, 96), (32, 2, 128), (20, 1, 64), (3, 3, 128)])
def test_tensor_core_attention_against_generic_and_plain(n_heads, n_kv, d):
    """The bf16 tensor-core kernels (prefill tiles, split-key decode) on sequences that end inside a
    page, at a page boundary and just after it; with history (chunked prompt) and without."""
    ops = _ops("bfloat16")
    lens = [1, 64, 65, 130, 333]
    cache, slots = _paged_setup(ops, lens, n_kv, d, 0, "bfloat16")
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(9)
    T = sum(lens)
    qkv = torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g).bfloat16()
    positions = torch.cat([torch.arange(n) for n in lens]).int().cuda()
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    sl = torch.tensor(slots, dtype=torch.int32).cuda()
    q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions, token_seq, sl, lane.page_table, lane.k, lane.v,
                       None, 1.0, 0)
    scale = 1 / math.sqrt(d)
    rows = qkv.float().view(T, n_heads + 2 * n_kv, d)
    want = torch.cat([plain.dense_attention(rows[o:o + n, :n_heads], rows[o:o + n, n_heads:n_heads + n_kv],
                                            rows[o:o + n, n_heads + n_kv:], scale).reshape(n, -1)
                      for o, n in zip([0, 1, 65, 130, 260], lens)])
    cu = torch.tensor([0, 1, 65, 130, 260, 593], dtype=torch.int32).cuda()
    kv_len = torch.tensor(lens, dtype=torch.int32).cuda()
    from cpmcu_b200.ops.ops import PREFILL_TILE_ROWS as TR
    tile_seq = [j for j, n in enumerate(lens) for _ in range(0, n, TR)]
    tile_row = [r for n in lens for r in range(0, n, TR)]
    tiles = (torch.tensor(tile_seq, dtype=torch.int32).cuda(), torch.tensor(tile_row, dtype=torch.int32).cuda(), len(tile_seq))
    got = ops.prefill_attention(q, lane.k, lane.v, tiles, cu, kv_len, sl, lane.page_table, n_kv, scale)
    assert _err(got, want) < KTOL["bfloat16"]
    generic = ops.attention_generic(q, lane.k, lane.v, positions, token_seq, sl, lane.page_table, n_kv, scale)
    assert _err(got, generic) < KTOL["bfloat16"]
    # the last 40 tokens of the longest sequence as a step of their own: the earlier ones are history
    o, n = 260, 333
    cu2 = torch.tensor([0, 40], dtype=torch.int32).cuda()
    tiles2 = (torch.zeros(1, dtype=torch.int32).cuda(), torch.zeros(1, dtype=torch.int32).cuda(), 1)
    got2 = ops.prefill_attention(q[o + n - 40:o + n].contiguous(), lane.k, lane.v, tiles2, cu2, kv_len[4:5].contiguous(),
                                 sl[4:5].contiguous(), lane.page_table, n_kv, scale)
    assert _err(got2, want[o + n - 40:o + n]) < KTOL["bfloat16"]
    # decode: the last token of every sequence, with few and with many shares
    last = torch.tensor([0, 64, 129, 259, 592])
    ql = q[last.cuda()].contiguous()
    for splits in (1, 3, 64, None):
        dec = ops.decode_attention(ql, lane.k, lane.v, kv_len, sl, lane.page_table, n_kv, scale, n_splits=splits)
        assert _err(dec, want[last]) < KTOL["bfloat16"], splits


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul_interleaved(dtype):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(10)
    inter = 88
    gate, up = torch.randn(5, inter, generator=g) * 2, torch.randn(5, inter, generator=g)
    gu = torch.stack([gate.view(5, inter // 8, 8), up.view(5, inter // 8, 8)], dim=2).reshape(5, 2 * inter).to(DT[dtype])
    got = ops.silu_mul(gu.cuda(), interleave=8)
    gf, uf = gate.to(DT[dtype]).float(), up.to(DT[dtype]).float()
    assert _err(got, gf * (1 / (1 + torch.exp(-gf))) * uf) < KTOL[dtype]


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 32), (48, 64), (1000, 128), (777, 96), (4608, 4096), (73448, 256)])
def test_skinny_gemm(M, N, K):
    """The weight-streaming product of the decode path against fp32 torch, all epilogues.  (The engine
    hands it up to 8 rows; the kernel takes up to 16, which is what the larger cases run.)"""
    ops = _ops("bfloat16")
    ops.SKINNY_MAX_ROWS = 16
    g = torch.Generator().manual_seed(11)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    want = a.float() @ w.float().T
    got = ops.linear(a.cuda(), w.cuda())
    assert got.dtype == torch.bfloat16 and _err(got, want) < KTOL["bfloat16"]
    got32 = ops.linear(a.cuda(), w.cuda(), alpha=0.125, out_f32=True)
    assert got32.dtype == torch.float32 and _err(got32, want * 0.125) < 2e-5
    if N % 16 == 0:
        inter = N // 2
        gate, up = w[:inter].float(), w[inter:].float()
        wi = torch.stack([w[:inter].view(inter // 8, 8, K), w[inter:].view(inter // 8, 8, K)], dim=1).reshape(N, K)
        gg, uu = a.float() @ gate.T, a.float() @ up.T
        h = ops.gated_linear(a.cuda(), wi.contiguous().cuda(), 8)
        assert _err(h, gg * (1 / (1 + torch.exp(-gg))) * uu) < KTOL["bfloat16"]
    # a row's result does not depend on the other rows
    one = ops.linear(a[:1].contiguous().cuda(), w.cuda(), out_f32=True, alpha=0.125)
    assert torch.equal(one[0], got32[0])


def test_which_products_of_9_to_16_rows_take_the_weight_streaming_kernel():
    """At 9 to 16 rows the engine keeps a product on the weight-streaming kernel while the bytes its blocks read of
    the activations stay small: the QKV, O and down products of the 8B sizes, not gate_up, the head or 17 rows."""
    ops = _ops("bfloat16")
    assert ops._skinny_ok(16, 4096, 4608) and ops._skinny_ok(9, 4096, 4096) and ops._skinny_ok(16, 14336, 4096)
    assert not ops._skinny_ok(16, 4096, 32768) and not ops._skinny_ok(16, 4096, 73448)
    assert not ops._skinny_ok(17, 4096, 4608) and ops._skinny_ok(8, 4096, 73448)


@pytest.mark.parametrize("tiles", ["no", "mma", "tcgen05"])
@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 1, 32), (6, 2, 64), (32, 2, 128), (20, 1, 64), (16, 1, 128)])
def test_block_list_attention_against_generic(n_heads, n_kv, d, tiles):
    """The bf16 block-list kernels against the generic kernel given the same lists: random subsets of
    pages that always hold the token's own page, and tokens whose list says "dense".  ``tiles``: the kernels in
    which consecutive tokens share the blocks that are brought ("mma": seven tokens on mma.sync; "tcgen05": eight
    tokens x sixteen heads as one tensor-core tile, which takes head size 128 with sixteen heads per key/value
    head and leaves the other shapes to the first); the sequences' ends (300, 364) fall inside tiles, so some
    tiles hold tokens of two sequences, and the longest sequence has more than 32 blocks (a second word of the
    block masks)."""
    from cpmcu_b200.ops import library
    ops = _ops("bfloat16")
    ops.use_tcgen05_listed = tiles == "tcgen05"
    lens = [300, 64, 2300]
    cache, slots = _paged_setup(ops, lens, n_kv, d, 0, "bfloat16")
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(12)
    T = sum(lens)
    qkv = torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g).bfloat16()
    positions = torch.cat([torch.arange(n) for n in lens]).int()
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    sl = torch.tensor(slots, dtype=torch.int32).cuda()
    q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions.cuda(), token_seq, sl, lane.page_table, lane.k, lane.v,
                       None, 1.0, 0)
    cap = 7
    lists = torch.full((T, n_kv, cap), -1, dtype=torch.int32)
    for t in range(T):
        own = int(positions[t]) // 64
        for h in range(n_kv):
            if t % 5 == 0:
                lists[t, h, 0] = -2
                continue
            others = torch.randperm(own, generator=g)[:min(own, 4)].tolist() if own > 0 else []
            blocks = sorted(set(others + [own]))
            lists[t, h, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
            lists[t, h, len(blocks) + 1:] = 12345                # what lies behind the terminator is not the list's
    lists = lists.cuda()
    scale = 1 / math.sqrt(d)
    want = ops.attention_generic(q, lane.k, lane.v, positions.cuda(), token_seq, sl, lane.page_table, n_kv, scale,
                                 block_list=lists, block_size=64)
    got = ops.listed_attention(q, lane.k, lane.v, positions.cuda(), token_seq, sl, lane.page_table, lists, n_kv, scale,
                               tiles=tiles != "no")
    ops.use_tcgen05_listed = True
    ops.raise_on_kernel_error()
    assert _err(got, want) < KTOL["bfloat16"]


def test_block_list_attention_of_random_batches():
    """The two tile kernels of the block-list attention on random batches: one to four sequences of lengths around
    the page and tile edges (so a tile holds tokens of up to four sequences, and unions of one, two, an odd and an
    even number of blocks all occur), one to three key/value heads, lists of 3, 7 and 40 places with any number of
    blocks in them, a fifth of the tokens "dense"."""
    import random
    ops = _ops("bfloat16")
    rnd = random.Random(5)
    d = 128
    try:
        for trial in range(16):
            n_kv = rnd.choice([1, 2, 3])
            n_heads = 16 * n_kv
            lens = [rnd.choice([1, 5, 63, 64, 65, 130, 300, 777, 1500]) for _ in range(rnd.randint(1, 4))]
            cache, slots = _paged_setup(ops, lens, n_kv, d, trial, "bfloat16")
            lane = cache.lane(0)
            g = torch.Generator().manual_seed(100 + trial)
            T = sum(lens)
            qkv = torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g).bfloat16()
            positions = torch.cat([torch.arange(n) for n in lens]).int()
            token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
            sl = torch.tensor(slots, dtype=torch.int32).cuda()
            q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions.cuda(), token_seq, sl, lane.page_table, lane.k,
                               lane.v, None, 1.0, 0)
            cap = rnd.choice([3, 7, 40])
            lists = torch.full((T, n_kv, cap), -1, dtype=torch.int32)
            for t in range(T):
                own = int(positions[t]) // 64
                for h in range(n_kv):
                    if rnd.random() < 0.2:
                        lists[t, h, 0] = -2
                        continue
                    k = rnd.randint(0, min(own, cap - 1))
                    blocks = sorted(set(rnd.sample(range(own), k) + [own]))
                    lists[t, h, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
                    lists[t, h, len(blocks) + 1:] = 12345
            lists = lists.cuda()
            scale = 1 / math.sqrt(d)
            want = ops.attention_generic(q, lane.k, lane.v, positions.cuda(), token_seq, sl, lane.page_table, n_kv, scale,
                                         block_list=lists, block_size=64)
            for tcgen05 in (True, False):
                ops.use_tcgen05_listed = tcgen05
                got = ops.listed_attention(q, lane.k, lane.v, positions.cuda(), token_seq, sl, lane.page_table, lists,
                                           n_kv, scale, tiles=True)
                ops.raise_on_kernel_error()
                assert _err(got, want) < KTOL["bfloat16"], (trial, tcgen05, lens, n_kv, cap)
    finally:
        ops.use_tcgen05_listed = True


@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 2, 128), (2, 1, 128), (32, 2, 128), (16, 2, 64), (4, 2, 64)])
def test_tcgen05_prefill_attention(n_heads, n_kv, d):
    """The tcgen05 prefill attention (head sizes 128 and 64, heads in pairs) against the plain implementation:
    sequences that end inside a page, at a page or tile boundary and just after it, pages in scrambled
    order, a chunk after a history; and one far key made to dominate a late query."""
    ops = _ops("bfloat16")
    lens = [1, 64, 128, 129, 300, 577]
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts.base import CacheNeeds
    cache = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d)], max_tokens=64 * 40, dtype=torch.bfloat16, device="cuda:0")
    junk = cache.open_sequences(3)
    for j, s_ in enumerate(junk):
        cache.reserve(s_, 64 * (j + 1))
    slots = cache.open_sequences(len(lens))
    cache.close_sequence(junk[1])
    for s_, n in zip(slots, lens):
        cache.reserve(s_, n)
        cache.set_length(s_, n)
    cache.sync()
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(11)
    T = sum(lens)
    starts = [sum(lens[:i]) for i in range(len(lens))]
    qkv = (torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g) * 0.5)
    rows = qkv.view(T, n_heads + 2 * n_kv, d)
    far_key, late = starts[5] + 70, starts[5] + 560                  # in the longest sequence
    rows[far_key, n_heads:n_heads + n_kv] = 2.0
    rows[late, :n_heads] = 2.0
    qkv = qkv.bfloat16()
    rows = qkv.float().view(T, n_heads + 2 * n_kv, d)
    positions = torch.cat([torch.arange(n) for n in lens]).int().cuda()
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    sl = torch.tensor(slots, dtype=torch.int32).cuda()
    q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions, token_seq, sl, lane.page_table, lane.k, lane.v,
                       None, 1.0, 0)
    scale = 1 / math.sqrt(d)
    want = torch.cat([plain.dense_attention(rows[o:o + n, :n_heads], rows[o:o + n, n_heads:n_heads + n_kv],
                                            rows[o:o + n, n_heads + n_kv:], scale).reshape(n, -1)
                      for o, n in zip(starts, lens)])
    cu = torch.tensor(starts + [T], dtype=torch.int32).cuda()
    kv_len = torch.tensor(lens, dtype=torch.int32).cuda()
    from cpmcu_b200.ops.ops import PREFILL_TILE_ROWS as TR
    tile_seq = [j for j, n in enumerate(lens) for _ in range(0, n, TR)]
    tile_row = [r for n in lens for r in range(0, n, TR)]
    tiles = (torch.tensor(tile_seq, dtype=torch.int32).cuda(), torch.tensor(tile_row, dtype=torch.int32).cuda(), len(tile_seq))
    got = ops.prefill_attention_tcgen05(q, lane.k, lane.v, tiles, cu, kv_len, sl, lane.page_table, n_kv, scale)
    assert ops.attention_tcgen05_error() == 0
    assert _err(got, want) < KTOL["bfloat16"]
    # the far key's value comes through at the late query
    v_far = rows[far_key, n_heads + n_kv]
    assert _err(got[late].view(n_heads, d)[0], v_far) < 2e-2
    # the last 150 tokens of the longest sequence as a step of their own: the earlier ones are history
    o, n = starts[5], lens[5]
    cu2 = torch.tensor([0, 150], dtype=torch.int32).cuda()
    tiles2 = (torch.zeros(3, dtype=torch.int32).cuda(), torch.tensor([0, 64, 128], dtype=torch.int32).cuda(), 3)
    got2 = ops.prefill_attention_tcgen05(q[o + n - 150:o + n].contiguous(), lane.k, lane.v, tiles2, cu2,
                                         kv_len[5:6].contiguous(), sl[5:6].contiguous(), lane.page_table, n_kv, scale)
    assert ops.attention_tcgen05_error() == 0
    assert _err(got2, want[o + n - 150:o + n]) < KTOL["bfloat16"]


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N,K", [(1, 8, 64), (128, 256, 64), (300, 264, 192), (129, 4608, 128), (2048, 352, 64),
                                   (777, 1024, 4096), (4500, 2560, 128)])
def test_tcgen05_gemm(M, N, K, pair):
    """The tcgen05 / TMA / TMEM product against fp32 torch: tiles that hang over the edge in M and in N,
    one and many K blocks, more tiles than one wave of blocks, more rows than one band of tiles, plain and
    gated epilogue; by single blocks and by pairs of blocks on one tile."""
    ops = _ops("bfloat16")
    g = torch.Generator().manual_seed(13)
    a = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    want = a.float() @ w.float().T
    got = ops.linear_tcgen05(a, w, pair=pair)
    assert ops.tcgen05_error() == 0
    assert _err(got, want) < KTOL["bfloat16"]
    if N % 32 == 0:
        inter = N // 2
        wi = torch.stack([w[:inter].view(inter // 8, 8, K), w[inter:].view(inter // 8, 8, K)], dim=1).reshape(N, K).contiguous()
        gate, up = a.float() @ w[:inter].float().T, a.float() @ w[inter:].float().T
        h = ops.linear_tcgen05(a, wi, gated=True, pair=pair)
        assert ops.tcgen05_error() == 0
        assert _err(h, gate * torch.sigmoid(gate) * up) < KTOL["bfloat16"]


@pytest.mark.parametrize("d", [128, 64])
def test_tcgen05_prefill_attention_rescales_and_long_history(d):
    """Scores that keep growing along the sequence, so that the running maximum of a row is raised again and
    again (the kernel then rescales its accumulator in tensor memory), over 3,000 keys; then a chunk of 200
    tokens whose history is the rest."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts.base import CacheNeeds
    from cpmcu_b200.ops.ops import PREFILL_TILE_ROWS as TR

    n_heads, n_kv, n = 2, 1, 3000
    ops = _ops("bfloat16")
    cache = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d)], max_tokens=64 * 50, dtype=torch.bfloat16, device="cuda:0")
    slot = cache.open_sequence()
    cache.reserve(slot, n)
    cache.set_length(slot, n)
    cache.sync()
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(17)
    qkv = torch.randn(n, (n_heads + 2 * n_kv) * d, generator=g)
    rows = qkv.view(n, n_heads + 2 * n_kv, d)
    direction = torch.randn(d, generator=g)
    direction /= direction.norm()
    # every query looks along ``direction``; the keys' component along it grows with the position, so the score of
    # the newest keys exceeds all earlier ones by more and more (about 0.12 * position / sqrt(d) * |q| in all)
    rows[:, :n_heads] = 0.3 * rows[:, :n_heads] + 6.0 * direction
    rows[:, n_heads:n_heads + n_kv] = 0.3 * rows[:, n_heads:n_heads + n_kv] + (torch.arange(n)[:, None, None] * 0.02) * direction
    qkv = qkv.bfloat16()
    rows = qkv.float().view(n, n_heads + 2 * n_kv, d)
    positions = torch.arange(n).int().cuda()
    token_seq = torch.zeros(n, dtype=torch.int32).cuda()
    sl = torch.tensor([slot], dtype=torch.int32).cuda()
    q = ops.rope_store(qkv.cuda(), n_heads, n_kv, d, positions, token_seq, sl, lane.page_table, lane.k, lane.v, None, 1.0, 0)
    scale = 1 / math.sqrt(d)
    want = plain.dense_attention(rows[:, :n_heads], rows[:, n_heads:n_heads + n_kv], rows[:, n_heads + n_kv:], scale).reshape(n, -1)
    # the row maximum in log2 units rises by far more than the kernel's rescaling threshold of 8 along a row
    s_last = (rows[n - 1, 0] @ rows[:, n_heads].T) * scale * 1.4427
    assert float(s_last[-1] - s_last[64]) > 30
    cu = torch.tensor([0, n], dtype=torch.int32).cuda()
    kv_len = torch.tensor([n], dtype=torch.int32).cuda()
    tile_row = list(range(0, n, TR))
    tiles = (torch.zeros(len(tile_row), dtype=torch.int32).cuda(), torch.tensor(tile_row, dtype=torch.int32).cuda(), len(tile_row))
    got = ops.prefill_attention_tcgen05(q, lane.k, lane.v, tiles, cu, kv_len, sl, lane.page_table, n_kv, scale)
    assert ops.attention_tcgen05_error() == 0
    assert _err(got, want) < KTOL["bfloat16"]
    tail = 200
    cu2 = torch.tensor([0, tail], dtype=torch.int32).cuda()
    tr2 = list(range(0, tail, TR))
    tiles2 = (torch.zeros(len(tr2), dtype=torch.int32).cuda(), torch.tensor(tr2, dtype=torch.int32).cuda(), len(tr2))
    for shares in (1, 2, 5, 16, 40):                               # the keys of a tile shared out over several blocks
        got2 = ops.prefill_attention_tcgen05(q[n - tail:].contiguous(), lane.k, lane.v, tiles2, cu2, kv_len, sl, lane.page_table,
                                             n_kv, scale, n_splits=shares)
        assert ops.attention_tcgen05_error() == 0
        assert _err(got2, want[n - tail:]) < KTOL["bfloat16"], shares
    # two tiles of 16 head pairs leave most SMs idle: the keys are shared out; a whole 2,048-token prompt is not
    assert 1 < ops.prefill_key_shares([tail], n, 32) <= ops.sm_count // 32 and ops.prefill_key_shares([2048], 2048, 32) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pool_keys_and_select_blocks(dtype):
    """InfLLM-v2 key pooling (in two steps, so that windows straddle the step boundary) and block selection for
    every query of a 700-token sequence, at sizes no test model has (head size 64, two key-value heads with four
    query heads each, windows of 16 keys every 8, blocks of 64, four blocks chosen, a local window of two): the
    pooled keys against the plain means, the block lists against the plain selection (in bf16 where the choice
    is not a near tie)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts import StepContext
    from cpmcu_b200.parts.base import CacheNeeds

    ops = _ops(dtype)
    n_heads, n_kv, d, n = 8, 2, 64, 700
    sparse = {"kernel_size": 16, "kernel_stride": 8, "block_size": 64, "init_blocks": 1, "topk": 4, "window_size": 128,
              "dense_len": 0}
    cache = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d, pooled_stride=8, pooled_kernel=16)], max_tokens=64 * 16,
                  dtype=DT[dtype], device="cuda:0")
    junk = cache.open_sequence()
    cache.reserve(junk, 130)                                 # so that logical and physical pages differ
    slot = cache.open_sequence()
    cache.reserve(slot, n)
    cache.sync()
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(23)
    qkv = torch.randn(n, (n_heads + 2 * n_kv) * d, generator=g).to(DT[dtype])
    rows = qkv.float().view(n, n_heads + 2 * n_kv, d)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    sl = i32([slot])
    q_all = []
    for lo, hi in ((0, 300), (300, n)):
        m = hi - lo
        ctx = StepContext(m, 1, False, False, [m], [hi], [slot], m, hi, i32([0] * m), i32(list(range(lo, hi))), i32([0] * m),
                          i32([0, m]), i32([hi]), sl, cache)
        q_all.append(ops.rope_store(qkv[lo:hi].cuda(), n_heads, n_kv, d, ctx.positions, ctx.token_seq, sl, lane.page_table,
                                    lane.k, lane.v, None, 1.0, 0))
        ops.pool_keys(ctx, lane, n_kv, d, 16, 8)
    want_ck = plain.compress_keys(rows[:, n_heads:n_heads + n_kv], 16, 8)            # [n_c, kv, d]
    n_c = want_ck.shape[0]
    pages = cache.groups[0].pages_of_slot[slot]
    stored = torch.stack([lane.pooled[pages[i // 8], :, i % 8].cpu() for i in range(n_c)])              # [n_c, kv, d] fp32
    if dtype == "bfloat16":
        # with a bf16 cache a pooled key lies in its d floats as two bf16 terms, d leading ones and d residuals
        terms = stored.contiguous().view(torch.bfloat16).view(n_c, n_kv, 2, d).float()
        got_ck = terms[:, :, 0] + terms[:, :, 1]
        assert _err(got_ck, want_ck) < 2e-5                  # the mean to 16 bits
    else:
        assert _err(stored, want_ck) < 1e-6                  # fp32
    ctx = StepContext(n, 1, False, False, [n], [n], [slot], n, n, i32([0] * n), i32(list(range(n))), i32([0] * n),
                      i32([0, n]), i32([n]), sl, cache)
    q = torch.cat(q_all)
    scale = 1 / math.sqrt(d)
    lists, bs = ops.select_blocks(ctx, q, lane, n_kv, scale, sparse)
    assert bs == 64
    lists = lists.cpu()
    checked = 0
    for p in range(n):
        margins = []
        want = plain.select_blocks(rows[p, :n_heads], want_ck, p, scale, sparse, margins)
        for j in range(n_kv):
            if dtype == "bfloat16" and margins[j] < 0.02:
                continue
            row = lists[p, j].tolist()                      # block ids up to the first negative entry
            got = sorted(row[:next((i for i, b in enumerate(row) if b < 0), len(row))])
            assert got == want[j], (p, j, got, want[j])
            checked += 1
    assert checked > (n * n_kv) * (0.99 if dtype == "float32" else 0.8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_select_blocks_at_long_context_sizes(dtype):
    """Block selection at the sizes of a long-context model: head size 128, sixteen query heads per key-value head,
    windows of 32 keys every 16, blocks of 64, 64 blocks chosen among about 600, a local window of 32 blocks, 40,960
    cached tokens.  Every block's keys lean along one direction by an amount of their own and the queries look along
    it, so that block scores are spread out and the choice is firm; queries are a sample of positions (the first
    sparse one, page and block edges, the last).  The launch is sized once by the longest sequence of the step and
    once, as inside a captured step, by the cache's capacity per sequence (here 524,288 tokens)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts import StepContext
    from cpmcu_b200.parts.base import CacheNeeds

    ops = _ops(dtype)
    n_heads, n_kv, d, n = 32, 2, 128, 40960
    sparse = {"kernel_size": 32, "kernel_stride": 16, "block_size": 64, "init_blocks": 1, "topk": 64,
              "window_size": 2048, "dense_len": 8192}
    cache = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d, pooled_stride=16, pooled_kernel=32)], max_tokens=n + 256,
                  dtype=DT[dtype], device="cuda:0", n_slots=3, max_seq_tokens=8 * 65536)
    junk = cache.open_sequence()
    cache.reserve(junk, 130)
    slot = cache.open_sequence()
    cache.reserve(slot, n)
    cache.sync()
    lane = cache.lane(0)
    g = torch.Generator().manual_seed(31)
    direction = torch.randn(n_kv, d, generator=g)
    direction /= direction.norm(dim=-1, keepdim=True)
    n_blocks = n // 64
    lean = (torch.rand(n_blocks, n_kv, generator=g) * 16 - 8)                      # per block and kv head
    k_all = 0.05 * torch.randn(n, n_kv, d, generator=g) + lean.repeat_interleave(64, dim=0)[:, :, None] * direction
    k_all = k_all.to(DT[dtype])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    sl = i32([slot])
    for lo in range(0, n, 4096):
        m = 4096
        qkv = torch.zeros(m, n_heads + 2 * n_kv, d, dtype=DT[dtype])
        qkv[:, n_heads:n_heads + n_kv] = k_all[lo:lo + m]
        ctx = StepContext(m, 1, False, False, [m], [lo + m], [slot], m, lo + m, i32([0] * m), i32(list(range(lo, lo + m))),
                          i32([0] * m), i32([0, m]), i32([lo + m]), sl, cache)
        ops.rope_store(qkv.view(m, -1).cuda(), n_heads, n_kv, d, ctx.positions, ctx.token_seq, sl, lane.page_table,
                       lane.k, lane.v, None, 1.0, 0)
        ops.pool_keys(ctx, lane, n_kv, d, 32, 16)
    ck = plain.compress_keys(k_all.float(), 32, 16)
    sample = sorted({8191, 8192, 8193, 8255, 8256, 10239, 10240, 16383, 16384, 30000, 32767, 32768, n - 65, n - 64, n - 1}
                    | set(torch.randint(8192, n, (33,), generator=g).tolist()))
    m = len(sample)
    q_rows = (0.05 * torch.randn(m, n_heads, d, generator=g)
              + 40.0 * direction.repeat_interleave(n_heads // n_kv, dim=0)[None]).to(DT[dtype])
    qkv = torch.zeros(m, n_heads + 2 * n_kv, d, dtype=DT[dtype])
    qkv[:, :n_heads] = q_rows
    scale = 1 / math.sqrt(d)
    all_sample, all_rows, all_qkv = sample, q_rows, qkv
    few = list(range(0, 6)) + list(range(len(sample) - 6, len(sample)))           # a dozen queries: the path for decode steps
    for captured, pick in ((False, None), (True, None), (False, few), (True, few)):
        sample = all_sample if pick is None else [all_sample[i] for i in pick]
        q_rows = all_rows if pick is None else all_rows[pick]
        qkv = all_qkv if pick is None else all_qkv[pick].contiguous()
        m = len(sample)
        longest = cache.max_pages_per_seq * 64 if captured else n       # a recorded step knows only the cache's capacity
        ctx = StepContext(m, 1, False, captured, [m], [n], [slot], m, longest, i32([0] * m), i32(sample), i32([0] * m),
                          i32([0, m]), i32([n]), sl, cache)
        q = ops.rope_store(qkv.view(m, -1).cuda(), n_heads, n_kv, d, ctx.positions, ctx.token_seq, sl, lane.page_table,
                           None, None, None, 1.0, 0)
        from cpmcu_b200.ops import library
        before = library.LAUNCHES[0]
        lists, bs = ops.select_blocks(ctx, q, lane, n_kv, scale, sparse)
        # few queries in bf16 share each query's pooled keys out over many blocks (two kernels instead of one)
        assert library.LAUNCHES[0] - before == (2 if pick is not None and dtype == "bfloat16" else 1)
        ops.raise_on_kernel_error()
        lists = lists.cpu()
        checked = 0
        for i, p in enumerate(sample):
            if p + 1 <= sparse["dense_len"]:
                assert lists[i, :, 0].tolist() == [-2] * n_kv                      # "dense": every key up to the query
                checked += n_kv
                continue
            margins = []
            want = plain.select_blocks(q_rows[i].float(), ck, p, scale, sparse, margins)
            for j in range(n_kv):
                if margins[j] < (1e-4 if dtype == "float32" else 5e-3):
                    continue
                row = lists[i, j].tolist()
                got = row[:next((x for x, b in enumerate(row) if b < 0), len(row))]
                assert got == want[j], (captured, p, j, got, want[j])
                assert len(got) == 64 + 32              # the leading block and 63 chosen ones, then the local window
                checked += 1
        assert checked >= 0.8 * m * n_kv, (checked, m * n_kv)


@pytest.mark.parametrize("M", [9, 17, 40, 64, 200])
def test_gated_product_of_a_decode_batch_takes_the_own_kernel(M):
    """9 to 255 rows (a decode batch) against a wide gate_up matrix: the gated product runs on the tcgen05 kernel
    with the activation in its epilogue (one launch of this library, no library product), against fp32 torch."""
    from cpmcu_b200.ops import library

    ops = _ops("bfloat16")
    inter, K = 9600, 128                                            # 75 tiles of 256 interleaved rows
    g = torch.Generator().manual_seed(19)
    a = torch.randn(M, K, generator=g).bfloat16().cuda()
    gate_w = (torch.randn(inter, K, generator=g) * 0.05).bfloat16().cuda()
    up_w = (torch.randn(inter, K, generator=g) * 0.05).bfloat16().cuda()
    wi = torch.stack([gate_w.view(inter // 8, 8, K), up_w.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    before = library.LAUNCHES[0]
    h = ops.gated_linear(a, wi, 8)
    assert library.LAUNCHES[0] - before == 1
    assert ops.tcgen05_error() == 0
    gate, up = a.float() @ gate_w.float().T, a.float() @ up_w.float().T
    assert _err(h, gate * torch.sigmoid(gate) * up) < KTOL["bfloat16"]


@pytest.mark.parametrize("n_heads,n_kv,d", [(32, 2, 128), (16, 2, 64), (6, 3, 128), (20, 1, 64)])
def test_decode_attention_with_rotation_inside(n_heads, n_kv, d):
    """The decode kernel that rotates q and the new key and stores the new key and value itself, against the
    rotary kernel followed by the plain decode kernel and against fp32 torch: the new token at the start, in the
    middle and at the end of a page, a sequence of one token, groups of more than 16 heads; afterwards both caches
    hold the same keys and values.  Also without rotation and without the store (a lane another run has written)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts.base import CacheNeeds

    ops = _ops("bfloat16")
    lens = [1, 64, 65, 300, 129, 640, 2, 191]                  # keys per sequence after this step
    g = torch.Generator().manual_seed(29)
    caches = [Cache([CacheNeeds(kv_heads=n_kv, head_dim=d)], max_tokens=64 * 40, dtype=torch.bfloat16, device="cuda:0")
              for _ in range(2)]
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
    mag = 1.1
    hist = [n - 1 for n in lens]
    T = sum(hist)
    old = torch.randn(T, (n_heads + 2 * n_kv) * d, generator=g).bfloat16().cuda()
    new = torch.randn(len(lens), (n_heads + 2 * n_kv) * d, generator=g).bfloat16().cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    slots_of = []
    for c in caches:                                          # the history, stored by the rotary kernel in both caches
        slots = c.open_sequences(len(lens))
        for s, n in zip(slots, lens):
            c.reserve(s, n)
        c.sync()
        lane = c.lane(0)
        pos = torch.cat([torch.arange(n) for n in hist]).int().cuda()
        seq = torch.cat([torch.full((n,), i) for i, n in enumerate(hist)]).int().cuda()
        ops.rope_store(old, n_heads, n_kv, d, pos, seq, i32(slots), lane.page_table, lane.k, lane.v, inv_freq, mag, d)
        slots_of.append(i32(slots))
    kv_len, scale = i32(lens), 1 / math.sqrt(d)
    seq = torch.arange(len(lens)).int().cuda()
    for splits in (None, 1, 3):
        a, b = caches[0].lane(0), caches[1].lane(0)
        q = ops.rope_store(new, n_heads, n_kv, d, i32(hist), seq, slots_of[0], a.page_table, a.k, a.v, inv_freq, mag, d)
        want = ops.decode_attention(q, a.k, a.v, kv_len, slots_of[0], a.page_table, n_kv, scale, n_splits=splits)
        got = ops.decode_attention_rope(new, b, kv_len, slots_of[1], n_heads, n_kv, d, scale, inv_freq, mag, True, n_splits=splits)
        assert _err(got, want) < 2e-3, splits             # same arithmetic; the rotation may round the last bit otherwise
        assert _err(b.k, a.k) < 1e-2 and torch.equal(b.v, a.v)
        # the lane is written already: only q comes from the product
        again = ops.decode_attention_rope(new, b, kv_len, slots_of[1], n_heads, n_kv, d, scale, inv_freq, mag, False, n_splits=splits)
        assert _err(again, want) < 2e-3
    # fp32 torch on the last sequence but one
    i = 5
    rows_old = old.float().cpu().view(T, n_heads + 2 * n_kv, d)[sum(hist[:i]):sum(hist[:i + 1])]
    rows = torch.cat([rows_old, new.float().cpu().view(len(lens), -1, d)[i:i + 1]])
    pos = torch.arange(lens[i])
    qr = plain.rotate(rows[:, :n_heads], pos, inv_freq.cpu(), mag)
    kr = plain.rotate(rows[:, n_heads:n_heads + n_kv], pos, inv_freq.cpu(), mag)
    ref = plain.dense_attention(qr, kr, rows[:, n_heads + n_kv:], scale)[-1].reshape(-1)
    assert _err(got[i], ref) < KTOL["bfloat16"]
    # no rotation at all (an encoding applied before, or none)
    c = Cache([CacheNeeds(kv_heads=n_kv, head_dim=d)], max_tokens=64 * 4, dtype=torch.bfloat16, device="cuda:0")
    s = c.open_sequence()
    c.reserve(s, 3)
    c.sync()
    lane = c.lane(0)
    three = torch.randn(3, (n_heads + 2 * n_kv) * d, generator=g).bfloat16().cuda()
    ops.rope_store(three[:2].contiguous(), n_heads, n_kv, d, i32([0, 1]), i32([0, 0]), i32([s]), lane.page_table, lane.k, lane.v, None, 1.0, 0)
    got = ops.decode_attention_rope(three[2:].contiguous(), lane, i32([3]), i32([s]), n_heads, n_kv, d, scale, None, 1.0, True)
    r3 = three.float().cpu().view(3, -1, d)
    ref = plain.dense_attention(r3[:, :n_heads], r3[:, n_heads:n_heads + n_kv], r3[:, n_heads + n_kv:], scale)[-1].reshape(-1)
    assert _err(got[0], ref) < KTOL["bfloat16"]
