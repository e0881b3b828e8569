"""The parts of a model alone, models put together from other parts than MiniCPM4's, and
schedules that run a layer twice or share a layer's keys and values.  Everything here is
built through the registries from a ModelSpec written in the test: no file of the
package is changed to add a part."""
import math

import pytest
import torch

from tests import configs, helpers
from tests.plain import minicpm4_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def _ops(dtype):
    from cpmcu_b200.ops.ops import Ops
    return Ops(DT[dtype], "cuda:0")


def _err(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


# ---------------------------------------------------------------------------
# each part alone
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from cpmcu_b200.parts import NORMS, PartSpec, build_part

    ops = _ops(dtype)
    norm = build_part(NORMS, PartSpec("rms_norm", {"hidden_size": 72, "eps": 3e-6}), ops)
    assert norm.weight_specs()["weight"].shape == (72,) and norm.weight_specs()["weight"].role == "vector"
    g = torch.Generator().manual_seed(0)
    w = (1 + 0.1 * torch.randn(72, generator=g)).to(DT[dtype])
    norm.load_weights({"weight": w.cuda()})
    x = torch.randn(11, 72, generator=g)
    assert _err(norm.forward(x.cuda()), plain.rms_norm(x, w.float(), 3e-6)) < TOL[dtype]
    d = torch.randn(11, 72, generator=g).to(DT[dtype])
    xs = x.clone().cuda()
    y = norm.add_forward(xs, d.cuda(), 0.7)
    assert _err(xs, x + 0.7 * d.float()) < 1e-6
    assert _err(y, plain.rms_norm(x + 0.7 * d.float(), w.float(), 3e-6)) < TOL[dtype]


def test_position_parts():
    from cpmcu_b200.parts import POSITIONS, PartSpec, build_part

    ops = _ops("float32")
    cfg = configs.tiny_b()
    rs = cfg["rope_scaling"]
    long = build_part(POSITIONS, PartSpec("longrope", {
        "head_dim": 32, "theta": cfg["rope_theta"], "long_factor": rs["long_factor"], "short_factor": rs["short_factor"],
        "original_max_positions": 64, "max_positions": 256}), ops)
    inv, mag, rot = long.rotary()
    want_inv, want_mag = plain.rope_table(cfg)
    assert rot == 32 and mag == pytest.approx(want_mag) and torch.equal(inv.cpu(), want_inv)
    short = build_part(POSITIONS, PartSpec("longrope", {
        "head_dim": 32, "theta": cfg["rope_theta"], "long_factor": rs["long_factor"], "short_factor": rs["short_factor"],
        "original_max_positions": 64, "max_positions": 64}), ops)
    inv_s, mag_s, _ = short.rotary()
    assert mag_s == 1.0 and torch.equal(inv_s.cpu(), plain.rope_table(dict(cfg, max_position_embeddings=64))[0])
    assert build_part(POSITIONS, PartSpec("none", {}), ops).rotary() == (None, 1.0, 0)
    with pytest.raises(KeyError, match="known"):
        build_part(POSITIONS, PartSpec("alibi", {}), ops)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter", [176, 100])          # a multiple of 8 (interleaved layout) and one that is not
def test_feed_forward_part(dtype, inter):
    from cpmcu_b200.parts import FEED_FORWARDS, PartSpec, build_part

    ops = _ops(dtype)
    ffn = build_part(FEED_FORWARDS, PartSpec("gated_ffn", {"hidden_size": 64, "intermediate_size": inter}), ops)
    g = torch.Generator().manual_seed(1)
    w = {n: (torch.randn(s.shape, generator=g) * 0.1).to(DT[dtype]) for n, s in ffn.weight_specs().items()}
    ffn.load_weights({n: t.cuda() for n, t in w.items()})
    for rows in (3, 40):                                # the decode product and the library product
        y = torch.randn(rows, 64, generator=g).to(DT[dtype])
        want = plain.gated_ffn(y.float(), {"p." + n: t.float() for n, t in w.items()}, "p.")
        assert _err(ffn.forward(None, y.cuda()), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from cpmcu_b200.parts import EMBEDDINGS, HEADS, PartSpec, build_part

    ops = _ops(dtype)
    emb = build_part(EMBEDDINGS, PartSpec("scaled_embedding", {"vocab_size": 777, "hidden_size": 72, "scale": 12.0}), ops)
    head = build_part(HEADS, PartSpec("scaled_lm_head", {"vocab_size": 777, "hidden_size": 72, "scale": 0.25, "tied": True}), ops)
    assert head.weight_specs() == {}
    g = torch.Generator().manual_seed(2)
    table = (torch.randn(777, 72, generator=g) * 0.02).to(DT[dtype])
    emb.load_weights({"weight": table.cuda()})
    head.tie(emb.weight)
    ids = [5, 776, 0, 5]
    assert _err(emb.forward(torch.tensor(ids, dtype=torch.int32).cuda()), plain.embed(ids, table.float(), 12.0)) < 1e-6
    y = torch.randn(4, 72, generator=g).to(DT[dtype])
    want = plain.lm_head(y.float(), {"model.embed_tokens.weight": table.float()}, {"tie_word_embeddings": True}, 0.25)
    got = head.forward(y.cuda())
    assert got.dtype == torch.float32 and _err(got, want) < TOL[dtype]


# ---------------------------------------------------------------------------
# a model from a hand-written specification, with a mixer the package does not know
# ---------------------------------------------------------------------------

def _register_toy_parts():
    from cpmcu_b200.parts import MIXERS, CacheNeeds, Mixer, WeightSpec

    if "toy_decay" in MIXERS:
        return

    @MIXERS.register("toy_decay")
    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + W_in y_t;  out_t = W_out s_t.  The running sum s is state of the
        mixer's own: one fp32 vector per sequence, kept by the cache beside the keys and values."""

        def __init__(self, ops, hidden_size, state_size, decay):
            super().__init__(ops)
            self.h, self.n, self.decay = hidden_size, state_size, decay

        def weight_specs(self):
            return {"in.weight": WeightSpec((self.n, self.h)), "out.weight": WeightSpec((self.h, self.n))}

        def load_weights(self, tensors):
            self.w_in, self.w_out = tensors["in.weight"].float(), tensors["out.weight"].float()

        def cache_needs(self):
            return CacheNeeds(state={"s": ((self.n,), torch.float32)})

        def forward(self, ctx, y, lane, writes_cache):
            out = torch.empty_like(y)
            state = lane.state["s"]
            o = 0
            for slot, n in zip(ctx.slots, ctx.q_lens):
                s = state[slot].clone()
                for t in range(n):
                    s = self.decay * s + self.w_in @ y[o + t].float()
                    out[o + t] = (self.w_out @ s).to(y.dtype)
                state[slot] = s
                o += n
            return out


TOY = dict(hidden=64, heads=4, kv=2, d=16, inter=96, vocab=300, eps=1e-5, state=24, decay=0.9, rs=0.8)


def _toy_spec(schedule=None):
    from cpmcu_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    _register_toy_parts()
    c = TOY
    norm = PartSpec("rms_norm", {"hidden_size": c["hidden"], "eps": c["eps"]})
    attn = PartSpec("gqa_attention", {"hidden_size": c["hidden"], "n_heads": c["heads"], "n_kv_heads": c["kv"],
                                      "head_dim": c["d"], "position": PartSpec("rope", {"head_dim": c["d"], "theta": 10000.0})})
    toy = PartSpec("toy_decay", {"hidden_size": c["hidden"], "state_size": c["state"], "decay": c["decay"]})
    ffn = PartSpec("gated_ffn", {"hidden_size": c["hidden"], "intermediate_size": c["inter"]})
    block = PartSpec("pre_norm_residual", {"residual_scale": c["rs"]})
    names = {"mixer_norm": "n1.", "mixer": "mix.", "feed_forward_norm": "n2.", "feed_forward": "ff."}
    layers = [LayerSpec(block, attn, ffn, norm, norm, "L0.", names), LayerSpec(block, toy, ffn, norm, norm, "L1.", names),
              LayerSpec(block, attn, ffn, norm, norm, "L2.", names)]
    if schedule is None:
        schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2)]
    return ModelSpec("Toy", c["hidden"], c["vocab"], PartSpec("scaled_embedding", {"vocab_size": c["vocab"], "hidden_size": c["hidden"], "scale": 3.0}),
                     layers, schedule, norm, PartSpec("scaled_lm_head", {"vocab_size": c["vocab"], "hidden_size": c["hidden"], "scale": 0.5}),
                     embedding_name="emb.", final_norm_name="fn.", head_name="head.")


def _toy_reference(w, ids, schedule):
    """The toy model with the plain implementation's functions; runs are (layer, lane, writes)."""
    c = TOY
    cfg = {"num_attention_heads": c["heads"], "num_key_value_heads": c["kv"], "head_dim": c["d"], "hidden_size": c["hidden"],
           "rope_theta": 10000.0, "max_position_embeddings": 4096}
    w = {k: v.float().cpu() for k, v in w.items()}
    S = len(ids)
    x = plain.embed(ids, w["emb.weight"], 3.0)
    lanes = {}
    for layer, lane, writes in schedule:
        p = f"L{layer}."
        y = plain.rms_norm(x, w[p + "n1.weight"], c["eps"])
        if layer == 1:
            s = torch.zeros(c["state"])
            a = torch.empty_like(y)
            for t in range(S):
                s = c["decay"] * s + w[p + "mix.in.weight"] @ y[t]
                a[t] = w[p + "mix.out.weight"] @ s
        else:
            a, kv = plain.attention_layer(y, w, p + "mix.", cfg, torch.arange(S), None if writes else lanes[lane])
            if writes:
                lanes[lane] = kv
        x = x + c["rs"] * a
        y = plain.rms_norm(x, w[p + "n2.weight"], c["eps"])
        ff = {"f.gate_proj.weight": w[p + "ff.gate_proj.weight"], "f.up_proj.weight": w[p + "ff.up_proj.weight"],
              "f.down_proj.weight": w[p + "ff.down_proj.weight"]}
        x = x + c["rs"] * plain.gated_ffn(y, ff, "f.")
    return plain.lm_head(plain.rms_norm(x, w["fn.weight"], c["eps"]), {"lm_head.weight": w["head.weight"]}, {}, 0.5)


def _toy_stepper(dtype, schedule=None):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.weights import random_tensors

    spec = _toy_spec(schedule)
    model = Model(spec, _ops(dtype))
    w = random_tensors(model.weight_specs(), 7, DT[dtype], std=0.1)
    model.load_weights({k: v.cuda() for k, v in w.items()})
    cache = Cache(model.cache_needs(), max_tokens=64 * 8, dtype=DT[dtype], device="cuda:0")
    return spec, w, Stepper(model, cache, chunk_tokens=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_of_its_own(dtype):
    from cpmcu_b200.engine import SequenceStep

    spec, w, st = _toy_stepper(dtype)
    sched = [(e.layer, e.lane, e.writes_cache) for e in spec.schedule]
    # the cache made a state tensor for the toy layer's lane, and no keys for it
    assert st.cache.lane(1).k is None and st.cache.lane(1).state["s"].shape[1] == TOY["state"]
    assert st.cache.lane(0).k is not None and st.cache.lane(0).state == {}
    seqs = [helpers.random_ids(TOY["vocab"], n, n) for n in (37, 5, 20)]
    wants = [_toy_reference(w, ids, sched) for ids in seqs]
    for round_ in range(2):                                    # the second round reuses the slots: state must restart
        slots = st.open(3)
        cut = [20, 5, 1]
        # prompts of unequal lengths in one step (chunked at 16 tokens), then token by token
        out = st.step([SequenceStep(s, ids[:c], list(range(c))) for s, ids, c in zip(slots, seqs, cut)])
        got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
        t = 0
        while any(c + t < len(ids) for ids, c in zip(seqs, cut)):
            live = [i for i in range(3) if cut[i] + t < len(seqs[i])]
            out = st.step([SequenceStep(slots[i], [seqs[i][cut[i] + t]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
            t += 1
        for i in range(3):
            assert _err(torch.cat(got[i]), wants[i]) < TOL[dtype], (round_, i)
            st.close(slots[i])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_runs_a_layer_twice_and_shares_a_cache_lane(dtype):
    """Order of layers is data: layer 0 runs twice (each run with a lane of its own), and layer 2
    reads the keys and values that the first run of layer 0 stored instead of making its own."""
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.parts import ScheduleEntry

    schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(2, 0, writes_cache=False)]
    spec, w, st = _toy_stepper(dtype, schedule)
    sched = [(e.layer, e.lane, e.writes_cache) for e in schedule]
    ids = helpers.random_ids(TOY["vocab"], 50, 3)
    want = _toy_reference(w, ids, sched)
    slot = st.open(1)[0]
    a = st.step([SequenceStep(slot, ids[:33], list(range(33)))])
    b = torch.cat([st.step([SequenceStep(slot, ids[i:i + 1], [0])]) for i in range(33, 50)])
    assert _err(torch.cat([a, b]), want) < TOL[dtype]
    from cpmcu_b200.models.model import Model
    with pytest.raises(ValueError, match="before any run has written"):
        Model(_toy_spec([ScheduleEntry(0, 1, writes_cache=False), ScheduleEntry(1, 1)]), _ops(dtype))


# ---------------------------------------------------------------------------
# places where a fault would hide
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model_folders, dtype):
    """300 tokens decoded one by one from a one-token prompt: every page boundary is crossed by a
    decode step, and the first tokens of the sequence are checked one by one."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import SequenceStep, Stepper
    from cpmcu_b200.loading import load_model

    folder = model_folders("tiny_c", configs.tiny_c(), 5, dtype)
    _, cfg, model = load_model(folder, dtype)
    st = Stepper(model, Cache(model.cache_needs(), 64 * 6, DT[dtype], "cuda:0"))
    ids = helpers.random_ids(cfg.vocab_size, 301, 9)
    want = helpers.plain_logits(folder, ids)
    slot = st.open(1)[0]
    rows = [st.step([SequenceStep(slot, ids[i:i + 1], [0])]) for i in range(301)]
    got = torch.cat(rows)
    for i in (0, 1, 2, 3):
        assert helpers.rel_err(got[i:i + 1], want[i:i + 1]) < helpers.TOL[dtype], i
    for lo in range(0, 301, 64):
        assert helpers.rel_err(got[lo:lo + 64], want[lo:lo + 64]) < helpers.TOL[dtype], lo


def test_window_attention_is_a_parameter_of_the_mixer():
    """A window of 24 keys on the attention part: its lanes form a cache group of their own."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts import MIXERS, PartSpec, StepContext, build_part

    ops = _ops("float32")
    spec = PartSpec("gqa_attention", {"hidden_size": 32, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "window": 24,
                                      "position": PartSpec("none", {})})
    att = build_part(MIXERS, spec, ops)
    full = build_part(MIXERS, PartSpec("gqa_attention", dict(spec.params, window=None)), ops)
    g = torch.Generator().manual_seed(4)
    w = {n: torch.randn(s.shape, generator=g) * 0.3 for n, s in att.weight_specs().items()}
    att.load_weights({n: t.cuda() for n, t in w.items()})
    full.load_weights({n: t.cuda() for n, t in w.items()})
    cache = Cache([att.cache_needs(), full.cache_needs()], 256, torch.float32, "cuda:0")
    assert len(cache.groups) == 2 and cache.groups[0].needs.window == 24 and cache.groups[1].needs.window is None
    slot = cache.open_sequence()
    n = 70
    cache.reserve(slot, n)
    cache.sync()
    y = torch.randn(n, 32, generator=g)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    ctx = StepContext(n, 1, False, False, [n], [n], [slot], n, n, i32([0] * n), i32(list(range(n))), i32([0] * n),
                      i32([0, n]), i32([n]), i32([slot]), cache)
    got = att.forward(ctx, y.cuda(), cache.lane(0), True)
    q = (y @ w["q_proj.weight"].T).view(n, 2, 16)
    k = (y @ w["k_proj.weight"].T).view(n, 1, 16)
    v = (y @ w["v_proj.weight"].T).view(n, 1, 16)
    want = plain.dense_attention(q, k, v, 0.25, window=24).reshape(n, 32) @ w["o_proj.weight"].T
    assert _err(got, want) < 2e-5
    dense = full.forward(ctx, y.cuda(), cache.lane(1), True)
    assert _err(dense[:24], want[:24]) < 2e-5 and _err(dense[30:], want[30:]) > 1e-3


def test_window_group_lets_pages_go_while_decoding():
    """The window part fed in steps (a chunk, then token by token, then chunks again): the pages of keys that
    have left the window go back to the pool on the way (the group holds a bounded number per sequence), a
    second sequence takes them over, and every output still equals the windowed plain attention."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.parts import MIXERS, PartSpec, StepContext, build_part

    ops = _ops("float32")
    window = 40
    spec = PartSpec("gqa_attention", {"hidden_size": 32, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "window": window,
                                      "position": PartSpec("none", {})})
    att = build_part(MIXERS, spec, ops)
    g = torch.Generator().manual_seed(5)
    w = {n: torch.randn(s.shape, generator=g) * 0.3 for n, s in att.weight_specs().items()}
    att.load_weights({n: t.cuda() for n, t in w.items()})
    step_tokens = 70
    cache = Cache([att.cache_needs()], 64 * 64, torch.float32, "cuda:0", n_slots=2, max_step_tokens=step_tokens)
    group = cache.groups[0]
    per_slot = (window + step_tokens + 63) // 64 + 1
    assert group.n_pages == 2 * per_slot                     # far fewer than the 64 pages of a group without window
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()

    def run(slot, y_all, cuts):
        outs, length = [], 0
        for n in cuts:
            cache.reserve(slot, length + n)
            cache.sync()
            ctx = StepContext(n, 1, n == 1, False, [n], [length + n], [slot], n, length + n, i32([0] * n),
                              i32(list(range(length, length + n))), i32([0] * n), i32([0, n]), i32([length + n]),
                              i32([slot]), cache)
            outs.append(att.forward(ctx, y_all[length:length + n].cuda(), cache.lane(0), True))
            length += n
            cache.set_length(slot, length)
            cache.check_consistent()
            assert group.pages_held(slot) <= per_slot
        return torch.cat(outs)

    def want_of(y):
        n = y.shape[0]
        q = (y @ w["q_proj.weight"].T).view(n, 2, 16)
        k = (y @ w["k_proj.weight"].T).view(n, 1, 16)
        v = (y @ w["v_proj.weight"].T).view(n, 1, 16)
        return plain.dense_attention(q, k, v, 0.25, window=window).reshape(n, 32) @ w["o_proj.weight"].T

    cuts = [70, 1, 1, 63] + [1] * 300 + [70, 5, 70]
    total = sum(cuts)
    y1, y2 = torch.randn(total, 32, generator=g), torch.randn(total, 32, generator=g)
    s1 = cache.open_sequence()
    got1 = run(s1, y1, cuts)
    assert _err(got1, want_of(y1)) < 2e-5
    assert total // 64 > group.n_pages                       # the sequence is longer than the whole group
    # a second sequence beside the first one: it gets pages that the first one has let go
    s2 = cache.open_sequence()
    got2 = run(s2, y2, cuts[::-1])
    assert _err(got2, want_of(y2)) < 2e-5
    cache.close_sequence(s1)
    cache.close_sequence(s2)
    assert group.pages.n_held == 0


# ---------------------------------------------------------------------------
# two more parts the package does not know: a feed-forward that routes each token to one of several small
# experts, and a position encoding that is not a rotation (it scales queries and keys by position)
# ---------------------------------------------------------------------------

def _register_routed_and_wave():
    from cpmcu_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, PositionEncoding, WeightSpec

    if "toy_routed" in FEED_FORWARDS:
        return

    @FEED_FORWARDS.register("toy_routed")
    class RoutedFeedForward(FeedForward):
        """out = p_e * W2_e relu(W1_e y) for the expert e with the largest router logit, p = softmax of the
        router logits (in 32-bit)."""

        def __init__(self, ops, hidden_size, expert_size, n_experts):
            super().__init__(ops)
            self.h, self.m, self.e = hidden_size, expert_size, n_experts

        def weight_specs(self):
            return {"router.weight": WeightSpec((self.e, self.h)), "w1": WeightSpec((self.e * self.m, self.h)),
                    "w2": WeightSpec((self.e * self.h, self.m))}

        def load_weights(self, tensors):
            self.router = tensors["router.weight"].float()
            self.w1 = tensors["w1"].view(self.e, self.m, self.h)
            self.w2 = tensors["w2"].view(self.e, self.h, self.m)

        def forward(self, ctx, y):
            logits = y.float() @ self.router.T
            p = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            out = torch.zeros_like(y)
            for e in range(self.e):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hid = torch.relu(self.ops.linear(y[rows].contiguous(), self.w1[e]))
                    out[rows] = (self.ops.linear(hid, self.w2[e]).float() * p[rows, e:e + 1]).to(y.dtype)
            return out

    @POSITIONS.register("toy_wave")
    class WavePosition(PositionEncoding):
        """q and k times (1 + amplitude * cos(position * rate_c)) per dimension c: not a rotation of pairs, so
        the attention part calls ``apply`` and stores the keys as they come out of it."""

        def __init__(self, ops, head_dim, amplitude):
            super().__init__(ops)
            self.rate = (0.1 * (1 + torch.arange(head_dim, dtype=torch.float32))).to(ops.device)
            self.amplitude = amplitude

        def apply(self, ctx, q, k):
            f = 1.0 + self.amplitude * torch.cos(ctx.positions.float()[:, None] * self.rate[None, :])
            q.mul_(f[:, None, :].to(q.dtype))
            k.mul_(f[:, None, :].to(k.dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(dtype):
    """A two-layer model whose feed-forwards route tokens to experts and whose attention uses a position
    encoding of the test's own: built from a specification, stepped in chunks and token by token, unequal
    batch, against a plain computation written here."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import SequenceStep, Stepper
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from cpmcu_b200.weights import random_tensors

    _register_routed_and_wave()
    H, heads, kv, d, vocab, eps, E, Msz, amp = 48, 3, 1, 16, 200, 1e-5, 3, 40, 0.3
    norm = PartSpec("rms_norm", {"hidden_size": H, "eps": eps})
    attn = PartSpec("gqa_attention", {"hidden_size": H, "n_heads": heads, "n_kv_heads": kv, "head_dim": d,
                                      "position": PartSpec("toy_wave", {"head_dim": d, "amplitude": amp})})
    ffn = PartSpec("toy_routed", {"hidden_size": H, "expert_size": Msz, "n_experts": E})
    dense = PartSpec("gated_ffn", {"hidden_size": H, "intermediate_size": 56})
    block = PartSpec("pre_norm_residual", {"residual_scale": 0.7})
    names = {"mixer_norm": "n1.", "mixer": "mix.", "feed_forward_norm": "n2.", "feed_forward": "ff."}
    layers = [LayerSpec(block, attn, ffn, norm, norm, "L0.", names), LayerSpec(block, attn, dense, norm, norm, "L1.", names)]
    spec = ModelSpec("Toy2", H, vocab, PartSpec("scaled_embedding", {"vocab_size": vocab, "hidden_size": H, "scale": 2.0}),
                     layers, [ScheduleEntry(0, 0), ScheduleEntry(1, 1)], norm,
                     PartSpec("scaled_lm_head", {"vocab_size": vocab, "hidden_size": H, "scale": 1.0}),
                     embedding_name="emb.", final_norm_name="fn.", head_name="head.")
    model = Model(spec, _ops(dtype))
    w = random_tensors(model.weight_specs(), 11, DT[dtype], std=0.15)
    model.load_weights({k: v.cuda() for k, v in w.items()})
    st = Stepper(model, Cache(model.cache_needs(), max_tokens=64 * 6, dtype=DT[dtype], device="cuda:0"), chunk_tokens=16)

    wf = {k: v.float().cpu() for k, v in w.items()}

    def reference(ids):
        """Returns the logits and, per position, how far the two best router logits are apart."""
        S = len(ids)
        pos = torch.arange(S, dtype=torch.float32)
        f = 1.0 + amp * torch.cos(pos[:, None] * (0.1 * (1 + torch.arange(d, dtype=torch.float32)))[None, :])
        x = plain.embed(ids, wf["emb.weight"], 2.0)
        margin = None
        for li in range(2):
            p = f"L{li}."
            y = plain.rms_norm(x, wf[p + "n1.weight"], eps)
            q = (y @ wf[p + "mix.q_proj.weight"].T).view(S, heads, d) * f[:, None, :]
            k = (y @ wf[p + "mix.k_proj.weight"].T).view(S, kv, d) * f[:, None, :]
            v = (y @ wf[p + "mix.v_proj.weight"].T).view(S, kv, d)
            a = plain.dense_attention(q, k, v, 1 / math.sqrt(d)).reshape(S, -1) @ wf[p + "mix.o_proj.weight"].T
            x = x + 0.7 * a
            y = plain.rms_norm(x, wf[p + "n2.weight"], eps)
            if li == 0:
                logits = y @ wf[p + "ff.router.weight"].T
                top = logits.topk(2, dim=-1).values
                margin = top[:, 0] - top[:, 1]
                prob = torch.softmax(logits, dim=-1)
                out = torch.zeros_like(y)
                for t in range(S):
                    e = int(logits[t].argmax())
                    w1 = wf[p + "ff.w1"].view(E, Msz, H)[e]
                    w2 = wf[p + "ff.w2"].view(E, H, Msz)[e]
                    out[t] = prob[t, e] * (w2 @ torch.relu(w1 @ y[t]))
                x = x + 0.7 * out
            else:
                ff = {"f.gate_proj.weight": wf[p + "ff.gate_proj.weight"], "f.up_proj.weight": wf[p + "ff.up_proj.weight"],
                      "f.down_proj.weight": wf[p + "ff.down_proj.weight"]}
                x = x + 0.7 * plain.gated_ffn(y, ff, "f.")
        return plain.lm_head(plain.rms_norm(x, wf["fn.weight"], eps), {"lm_head.weight": wf["head.weight"]}, {}, 1.0), margin

    seqs = [helpers.random_ids(vocab, n, 40 + n) for n in (41, 7, 23)]
    refs = [reference(ids) for ids in seqs]
    slots = st.open(3)
    cut = [30, 7, 2]
    out = st.step([SequenceStep(s, ids[:c], list(range(c))) for s, ids, c in zip(slots, seqs, cut)])
    got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
    t = 0
    while any(c + t < len(ids) for ids, c in zip(seqs, cut)):
        live = [i for i in range(3) if cut[i] + t < len(seqs[i])]
        out = st.step([SequenceStep(slots[i], [seqs[i][cut[i] + t]], [0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
        t += 1
    for i in range(3):
        g_all, (want, margin) = torch.cat(got[i]), refs[i]
        # in bf16 a router decision with two nearly equal logits may fall the other way: compare where it is firm
        firm = margin > (0.0 if dtype == "float32" else 0.05)
        assert int(firm.sum()) >= len(seqs[i]) // 2
        # a flipped decision changes the later positions of that sequence too (through attention): stop there
        upto = len(seqs[i]) if bool(firm.all()) else int((~firm).nonzero()[0])
        assert upto == len(seqs[i]) or dtype == "bfloat16"
        if upto:
            assert _err(g_all[:upto], want[:upto]) < TOL[dtype], i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_of_a_mixer_alone(dtype):
    """A layer needs no feed-forward: layer 0 is attention only (no feed-forward, no second norm, no tensors for
    them), layer 1 a whole layer; prompt in chunks, then token by token, against a plain computation."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import SequenceStep, Stepper
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from cpmcu_b200.weights import random_tensors

    c = TOY
    norm = PartSpec("rms_norm", {"hidden_size": c["hidden"], "eps": c["eps"]})
    attn = PartSpec("gqa_attention", {"hidden_size": c["hidden"], "n_heads": c["heads"], "n_kv_heads": c["kv"],
                                      "head_dim": c["d"], "position": PartSpec("rope", {"head_dim": c["d"], "theta": 10000.0})})
    ffn = PartSpec("gated_ffn", {"hidden_size": c["hidden"], "intermediate_size": c["inter"]})
    block = PartSpec("pre_norm_residual", {"residual_scale": c["rs"]})
    names = {"mixer_norm": "n1.", "mixer": "mix.", "feed_forward_norm": "n2.", "feed_forward": "ff."}
    layers = [LayerSpec(block, attn, None, norm, None, "L0.", names), LayerSpec(block, attn, ffn, norm, norm, "L1.", names)]
    spec = ModelSpec("MixerOnly", c["hidden"], c["vocab"],
                     PartSpec("scaled_embedding", {"vocab_size": c["vocab"], "hidden_size": c["hidden"], "scale": 3.0}),
                     layers, [ScheduleEntry(0, 0), ScheduleEntry(1, 1)], norm,
                     PartSpec("scaled_lm_head", {"vocab_size": c["vocab"], "hidden_size": c["hidden"], "scale": 0.5}),
                     embedding_name="emb.", final_norm_name="fn.", head_name="head.")
    model = Model(spec, _ops(dtype))
    assert not any(n.startswith("L0.ff.") or n.startswith("L0.n2.") for n in model.weight_specs())
    w = random_tensors(model.weight_specs(), 9, DT[dtype], std=0.1)
    model.load_weights({k: v.cuda() for k, v in w.items()})
    st = Stepper(model, Cache(model.cache_needs(), max_tokens=64 * 4, dtype=DT[dtype], device="cuda:0"), chunk_tokens=16)
    ids = helpers.random_ids(c["vocab"], 45, 4)
    wf = {k: v.float().cpu() for k, v in w.items()}
    cfg = {"num_attention_heads": c["heads"], "num_key_value_heads": c["kv"], "head_dim": c["d"], "hidden_size": c["hidden"],
           "rope_theta": 10000.0, "max_position_embeddings": 4096}
    x = plain.embed(ids, wf["emb.weight"], 3.0)
    for layer in (0, 1):
        p = f"L{layer}."
        a, _ = plain.attention_layer(plain.rms_norm(x, wf[p + "n1.weight"], c["eps"]), wf, p + "mix.", cfg, torch.arange(len(ids)))
        x = x + c["rs"] * a
        if layer == 1:
            y = plain.rms_norm(x, wf[p + "n2.weight"], c["eps"])
            x = x + c["rs"] * plain.gated_ffn(y, {"f." + n: wf[p + "ff." + n] for n in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")}, "f.")
    want = plain.lm_head(plain.rms_norm(x, wf["fn.weight"], c["eps"]), {"lm_head.weight": wf["head.weight"]}, {}, 0.5)
    slot = st.open(1)[0]
    got = [st.step([SequenceStep(slot, ids[:40], list(range(40)))])]
    got += [st.step([SequenceStep(slot, ids[i:i + 1], [0])]) for i in range(40, 45)]
    assert _err(torch.cat(got), want) < TOL[dtype]
