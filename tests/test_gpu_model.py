"""The engine against the plain implementation, through the step function: whole
sequences, the last tokens one by one, chunked prompts, and batches of unequal lengths
one after another so that slots and pages are used again.  float32 and bfloat16."""
import pytest
import torch

from tests import configs, helpers

pytestmark = pytest.mark.gpu

CASES = [
    ("tiny_a", configs.tiny_a, 0),
    ("tiny_b_dense", lambda: configs.tiny_b(sparse=False), 1),
    ("tiny_b", configs.tiny_b, 1),
    ("tiny_c", configs.tiny_c, 5),
    ("tiny_e", configs.tiny_e, 6),
]
DTYPES = ["float32", "bfloat16"]


def _stepper(folder, dtype, max_tokens=2048, chunk_tokens=2048):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.loading import load_model

    _, cfg, model = load_model(folder, dtype)
    cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=model.ops.dtype, device="cuda:0")
    st = Stepper(model, cache, chunk_tokens=chunk_tokens)
    helpers.record_blocks(st)        # sparse attention leaves its block choices, so that bf16 rows are all compared
    return cfg, st


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,make,seed", CASES)
def test_whole_sequence(model_folders, name, make, seed, dtype):
    from cpmcu_b200.engine import SequenceStep

    folder = model_folders(name, make(), seed, dtype)
    cfg, st = _stepper(folder, dtype)
    for n in (1, 5, 70, 150):
        ids = helpers.random_ids(cfg.vocab_size, n, seed + n)
        slot = st.open(1)[0]
        got = st.step([SequenceStep(slot, ids, list(range(n)))])
        st.close(slot)
        helpers.check_rows(got, folder, ids, range(n), dtype, (name, n), blocks=helpers.taken_blocks(st, slot))
    st.cache.check_consistent()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,make,seed", CASES)
def test_last_tokens_one_by_one(model_folders, name, make, seed, dtype):
    from cpmcu_b200.engine import SequenceStep

    folder = model_folders(name, make(), seed, dtype)
    cfg, st = _stepper(folder, dtype)
    n, tail = 150, 32
    ids = helpers.random_ids(cfg.vocab_size, n, seed + 100)
    slot = st.open(1)[0]
    rows = [st.step([SequenceStep(slot, ids[:n - tail], list(range(n - tail)))])]
    for i in range(n - tail, n):
        rows.append(st.step([SequenceStep(slot, ids[i:i + 1], [0])]))
    st.close(slot)
    got = torch.cat(rows)
    blocks = helpers.taken_blocks(st, slot)
    for lo, hi, what in ((0, n - tail, "prompt"), (n - tail, n, "decoded")):
        helpers.check_rows(got[lo:hi], folder, ids, range(lo, hi), dtype, (name, what), blocks=blocks)
    if dtype == "float32":
        helpers.check_rows(got[n - tail:n - tail + 1], folder, ids, [n - tail], dtype, (name, "first decoded"))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [7, 64])
def test_chunked_prompt(model_folders, dtype, chunk):
    from cpmcu_b200.engine import SequenceStep

    folder = model_folders("tiny_a", configs.tiny_a(), 0, dtype)
    cfg, st = _stepper(folder, dtype, chunk_tokens=chunk)
    lens = [33, 1, 130]
    seqs = [helpers.random_ids(cfg.vocab_size, n, 40 + n) for n in lens]
    slots = st.open(len(seqs))
    got = st.step([SequenceStep(s, ids, [len(ids) - 1, 0]) for s, ids in zip(slots, seqs)])
    k = 0
    for ids in seqs:
        want = helpers.plain_logits(folder, ids)
        assert helpers.rel_err(got[k:k + 1], want[-1:]) < helpers.TOL[dtype]
        assert helpers.rel_err(got[k + 1:k + 2], want[:1]) < helpers.TOL[dtype]
        k += 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,make,seed", CASES)
def test_unequal_batches_reuse_slots(model_folders, name, make, seed, dtype):
    """Batches of unequal prompts decode together; shorter requests end earlier; the next
    batch takes over their slots and pages with the old contents still in them."""
    from cpmcu_b200.engine import SequenceStep

    folder = model_folders(name, make(), seed, dtype)
    cfg, st = _stepper(folder, dtype, max_tokens=64 * 12)
    batches = [[(5, 3), (17, 20), (33, 9)], [(1, 24), (40, 2), (97, 11), (70, 16)], [(64, 5), (63, 70)]]
    for b, batch in enumerate(batches):
        seqs = [helpers.random_ids(cfg.vocab_size, p + d, 1000 * b + 10 * i + seed) for i, (p, d) in enumerate(batch)]
        slots = st.open(len(batch))
        got = [[] for _ in batch]
        taken = [None] * len(batch)
        out = st.step([SequenceStep(slots[i], seqs[i][:p], [p - 1]) for i, (p, d) in enumerate(batch)])
        for i in range(len(batch)):
            got[i].append(out[i])
        live = list(range(len(batch)))
        t = 0
        while live:
            live = [i for i in live if t < batch[i][1]]
            for i in range(len(batch)):
                if i not in live and slots[i] is not None and t >= batch[i][1]:
                    taken[i] = helpers.taken_blocks(st, slots[i])
                    st.close(slots[i])
                    slots[i] = None
            if not live:
                break
            out = st.step([SequenceStep(slots[i], [seqs[i][batch[i][0] + t]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r])
            t += 1
        for i, (p, d) in enumerate(batch):
            helpers.check_rows(torch.stack(got[i]), folder, seqs[i], range(p - 1, p + d), dtype, (name, b, i),
                               blocks=taken[i])
        st.cache.check_consistent()
    assert st.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_page_sized_sparse_blocks(model_folders, dtype):
    """Tiny D: prompts far beyond dense_len, whole, then decoded, in a batch of unequal lengths.
    The weights are drawn wider than usual (std 0.08) so that dropping the wrong block shows."""
    from cpmcu_b200.engine import SequenceStep

    folder = model_folders("tiny_d", configs.tiny_d(), 3, dtype, std=0.08)
    cfg, st = _stepper(folder, dtype, max_tokens=64 * 24)
    seqs = [helpers.random_ids(cfg.vocab_size, n, 50 + n) for n in (420, 130, 64)]
    slots = st.open(3)
    cut = [400, 101, 10]
    out = st.step([SequenceStep(s, ids[:c], list(range(c))) for s, ids, c in zip(slots, seqs, cut)])
    got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
    t = 0
    while any(c + t < len(ids) for ids, c in zip(seqs, cut)):
        live = [i for i in range(3) if cut[i] + t < len(seqs[i])]
        o = st.step([SequenceStep(slots[i], [seqs[i][cut[i] + t]], [0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(o[r:r + 1])
        t += 1
    for i, ids in enumerate(seqs):
        # every row in both precisions; in bfloat16 the plain implementation attends to the blocks the engine chose,
        # and each choice must be the rule's own up to rounding
        helpers.check_rows(torch.cat(got[i]), folder, ids, range(len(ids)), dtype, i, blocks=helpers.taken_blocks(st, slots[i]))
    # the sparse rule matters for this model: dense attention gives other logits for the long sequence
    cfgd, w = helpers.read_folder(folder)
    from tests.plain import minicpm4_plain as plain
    dense = plain.forward(dict(cfgd, sparse_config=None), w, seqs[0])
    assert helpers.rel_err(dense[300:], helpers.plain_logits(folder, seqs[0])[300:]) > 5 * helpers.TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_through_the_tcgen05_kernels(model_folders, dtype):
    """Head size 128 and prompts of 300 and more tokens: in bf16 the prompt goes through the tcgen05 attention
    and the tcgen05 gated product (both from their own size limits on), whole, in chunks of 128 with the
    history growing, two unequal prompts in one step, and then token by token through the decode kernels."""
    from cpmcu_b200.engine import SequenceStep

    folder = model_folders("tiny_e", configs.tiny_e(), 6, dtype)
    cfg, st = _stepper(folder, dtype, max_tokens=4096)
    a = helpers.random_ids(cfg.vocab_size, 420, 61)
    b = helpers.random_ids(cfg.vocab_size, 300, 62)
    want_rows = [0, 1, 127, 128, 255, 256, 299]
    s1, s2 = st.open(2)
    got = st.step([SequenceStep(s1, a[:400], want_rows + [399]), SequenceStep(s2, b, want_rows)])
    helpers.check_rows(got[:8], folder, a, want_rows + [399], dtype, "a whole")
    helpers.check_rows(got[8:], folder, b, want_rows, dtype, "b whole")
    tail = torch.cat([st.step([SequenceStep(s1, a[i:i + 1], [0])]) for i in range(400, 420)])
    helpers.check_rows(tail, folder, a, range(400, 420), dtype, "a decoded")
    st.close(s1)
    st.close(s2)
    _, st2 = _stepper(folder, dtype, max_tokens=4096, chunk_tokens=128)
    s3 = st2.open(1)[0]
    got = st2.step([SequenceStep(s3, a[:400], want_rows + [399])])
    helpers.check_rows(got, folder, a, want_rows + [399], dtype, "a in chunks")
    st2.close(s3)
    st.ops.raise_on_kernel_error()
    st.cache.check_consistent()


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_configurations(tmp_path, dtype):
    """A dozen configurations drawn at random (head sizes in steps of 16 up to 160, one to three key-value
    heads with one to eight query heads each, widths and vocabularies that are no power of two, one to three
    layers, tied or untied head): a prompt, chunked or whole, then five tokens one by one, against the plain
    implementation."""
    import random

    from cpmcu_b200.engine import SequenceStep

    rng = random.Random(20)
    for case in range(12):
        d = rng.choice([16, 32, 48, 64, 80, 96, 128, 160])
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 3, 4, 8])
        hidden = rng.choice([40, 64, 72, 96, 128, 200, 256])
        vocab = rng.choice([97, 300, 777, 1024])
        cfgd = {"architectures": ["MiniCPMForCausalLM"], "num_hidden_layers": rng.choice([1, 2, 3]), "hidden_size": hidden,
                "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": d,
                "intermediate_size": rng.choice([24, 56, 100, 176, 320]), "vocab_size": vocab,
                "max_position_embeddings": 4096, "rms_norm_eps": rng.choice([1e-5, 1e-6]),
                "rope_theta": rng.choice([1e4, 1e6]), "scale_emb": rng.choice([1, 7]),
                "dim_model_base": rng.choice([hidden, 32]), "scale_depth": rng.choice([1.0, 1.4]),
                "tie_word_embeddings": rng.choice([True, False])}
        n = rng.choice([3, 70, 200, 330])
        folder = helpers.make_folder(cfgd, str(tmp_path / f"c{case}"), case, dtype, std=0.05)
        cfg, st = _stepper(folder, dtype, max_tokens=1024, chunk_tokens=rng.choice([64, 2048]))
        ids = helpers.random_ids(vocab, n, case)
        slot = st.open(1)[0]
        cut = max(1, n - 5)
        rows = [st.step([SequenceStep(slot, ids[:cut], list(range(cut)))])]
        for i in range(cut, n):
            rows.append(st.step([SequenceStep(slot, ids[i:i + 1], [0])]))
        helpers.check_rows(torch.cat(rows), folder, ids, range(n), dtype, (case, cfgd))
        st.ops.raise_on_kernel_error()


@pytest.mark.parametrize("name,make,seed", [("tiny_e", configs.tiny_e, 6), ("tiny_f", configs.tiny_f, 7)])
def test_short_chunks_after_a_long_history(model_folders, name, make, seed):
    """A prompt of 2,300 tokens in chunks of 256 (bf16): from 1,024 keys on the head-size-64 model changes to the
    tcgen05 attention, and from 2,048 keys on the keys of a chunk's tiles are shared out over several blocks and
    combined by a second kernel.  Logits at places spread over the prompt, then ten decoded tokens."""
    from cpmcu_b200.engine import SequenceStep

    dtype = "bfloat16"
    folder = model_folders(name, make(), seed, dtype)
    cfg, st = _stepper(folder, dtype, max_tokens=4096, chunk_tokens=256)
    n = 2300
    ids = helpers.random_ids(cfg.vocab_size, n + 10, 70 + seed)
    places = [0, 255, 256, 1023, 1024, 1279, 2047, 2048, 2100, 2299]
    assert st.ops.prefill_key_shares([256], 2304, cfg.num_attention_heads) > 1
    slot = st.open(1)[0]
    got = st.step([SequenceStep(slot, ids[:n], places)])
    helpers.check_rows(got, folder, ids, places, dtype, (name, "prompt"))
    tail = torch.cat([st.step([SequenceStep(slot, ids[i:i + 1], [0])]) for i in range(n, n + 10)])
    helpers.check_rows(tail, folder, ids, range(n, n + 10), dtype, (name, "decoded"))
    st.close(slot)
    st.ops.raise_on_kernel_error()


@pytest.mark.parametrize("name,make,seed,dtype", [("tiny_a", configs.tiny_a, 0, "float32"), ("tiny_a", configs.tiny_a, 0, "bfloat16"),
                                                  ("tiny_b", configs.tiny_b, 1, "float32"), ("tiny_e", configs.tiny_e, 6, "bfloat16"),
                                                  ("tiny_f", configs.tiny_f, 7, "bfloat16")])
def test_full_prompt_chunks_through_a_recorded_graph(model_folders, name, make, seed, dtype):
    """Prompts of several chunks with the chunk graph on: the first full chunk runs the ordinary way and is recorded,
    the later ones (other histories, another sequence in another slot, a reused slot) are replays; the last, partial
    chunk and the decode steps run the ordinary way again.  Logits at places in every chunk against the plain
    implementation."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import SequenceStep, Stepper
    from cpmcu_b200.loading import load_model

    folder = model_folders(name, make(), seed, dtype)
    _, cfg, model = load_model(folder, dtype)
    chunk = 64
    cache = Cache(model.cache_needs(), max_tokens=64 * 24, dtype=model.ops.dtype, device="cuda:0", max_step_tokens=chunk)
    st = Stepper(model, cache, chunk_tokens=chunk, graph_prompts=True)
    assert st.graph_prompts
    limit = min(cfg.max_position_embeddings, 330) if name != "tiny_a" else 120
    for pass_, n in enumerate((limit, limit - 70, limit - 3)):
        ids = helpers.random_ids(cfg.vocab_size, n + 3, 300 + pass_)
        places = sorted(p for p in {0, 5, 63, 64, 65, 127, 128, n // 2, n - 2, n - 1} if p < n)
        slot = st.open(1)[0]
        got = st.step([SequenceStep(slot, ids[:n], places)])
        helpers.check_rows(got, folder, ids, places, dtype, (name, pass_, "prompt"))
        tail = torch.cat([st.step([SequenceStep(slot, ids[i:i + 1], [0])]) for i in range(n, n + 3)])
        helpers.check_rows(tail, folder, ids, range(n, n + 3), dtype, (name, pass_, "decoded"))
        if pass_ != 1:
            st.close(slot)                                    # the third pass runs beside the second pass's sequence, in another slot
    assert len(st.prompt_graphs) >= 1 and all(k[0] == chunk and k[2] == 1024 for k in st.prompt_graphs)
    st.ops.raise_on_kernel_error()
    # a model with a part that reads the batch on the host keeps to the ordinary way
    from tests import toy_arch  # noqa: F401  (registers the architecture)
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.registry import architecture
    toy = architecture(toy_arch.NAME)
    assert not Model(toy.model_spec(toy.config_class.from_dict(toy_arch.config_dict())), None).recordable_prompt()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hd64", "hd128"])
def test_engine_against_the_reference_golden(tmp_path, name, dtype):
    """The engine's logits against those the unmodified reference produced for the same tiny random model
    (tests/golden, made on a GPU by tests/golden/make_reference_golden.py): the prompt in chunks of 32 tokens as
    the reference ran it, then tokens one by one, in fp32 and in bf16.  The reference computed in bf16."""
    import json
    import os

    import numpy as np
    from safetensors.torch import save_file

    from cpmcu_b200.engine import SequenceStep
    from tests.golden import make_reference_golden as golden

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", f"reference_{name}.npz"))
    cfg = json.loads(str(data["config"]))
    ids, positions = data["ids"].tolist(), data["positions"].tolist()
    want = torch.from_numpy(data["logits"])
    folder = str(tmp_path / name)
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(cfg, architectures=["MiniCPMForCausalLM"], model_type="minicpm", torch_dtype="bfloat16"), f)
    save_file(golden.make_weights(cfg, int(data["seed"])), os.path.join(folder, "model.safetensors"))
    _, st = _stepper(folder, dtype, chunk_tokens=32)
    slot = st.open(1)[0]
    prompt = golden.PROMPT
    rows = {}
    wanted = [p for p in positions if p < prompt]
    got = st.step([SequenceStep(slot, ids[:prompt], wanted)])
    for p, row in zip(wanted, got):
        rows[p] = row
    for at in range(prompt, len(ids)):
        rows[at] = st.step([SequenceStep(slot, [ids[at]], [0])])[0]
    st.close(slot)
    got = torch.stack([rows[p] for p in positions]).float().cpu()
    err = float((got - want).abs().max() / want.abs().max())
    assert err < 2e-2, (name, dtype, err)
    top2 = want.topk(2, dim=-1).values
    firm = (top2[:, 0] - top2[:, 1]) > 4e-2 * float(want.abs().max())
    assert torch.equal(got.argmax(-1)[firm], want.argmax(-1)[firm])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,make,seed", [("tiny_a", configs.tiny_a, 1), ("tiny_e", configs.tiny_e, 6), ("tiny_f", configs.tiny_f, 7)])
def test_packed_chunks_through_a_recorded_graph(model_folders, name, make, seed, dtype):
    """A batch of unequal prompts in chunks of 128 packed tokens: full chunks hold pieces of several sequences
    (58 tokens of one, then 70 of the next, ...) and are recorded into graphs the first time their kind runs.  Three
    batches with other tokens and other lengths: the first records as it goes, the others replay; every wanted
    row is compared with the plain implementation.  Unused query tiles and sequences of the recorded shape are
    empty ones."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import SequenceStep, Stepper
    from cpmcu_b200.loading import load_model

    folder = model_folders(name, make(), seed, dtype)
    _, cfg, model = load_model(folder, dtype)
    limit = min(cfg.max_position_embeddings, 230)
    cache = Cache(model.cache_needs(), max_tokens=4096, dtype=model.ops.dtype, device="cuda:0")
    st = Stepper(model, cache, chunk_tokens=128, graph_prompts=True)
    replayed = 0
    for pass_, lens in enumerate(([70, 130, 40, limit, 90], [128, 60, limit, 33, 100, 64], [limit, 5, 200, 120, 70])):
        lens = [min(n, limit) for n in lens]
        seqs = [helpers.random_ids(cfg.vocab_size, n, 500 + 10 * pass_ + k) for k, n in enumerate(lens)]
        slots = st.open(len(lens))
        wants = [sorted({0, n // 2, n - 1}) for n in lens]
        before = len(st.prompt_graphs)
        got = st.step([SequenceStep(s, ids, w) for s, ids, w in zip(slots, seqs, wants)])
        replayed += before
        at = 0
        for k, (ids, w) in enumerate(zip(seqs, wants)):
            helpers.check_rows(got[at:at + len(w)], folder, ids, w, dtype, (name, pass_, k))
            at += len(w)
        tail = st.step([SequenceStep(s, [7], [0]) for s in slots])                  # and the cache is whole: one more token each
        for k, ids in enumerate(seqs):
            helpers.check_rows(tail[k:k + 1], folder, list(ids) + [7], [len(ids)], dtype, (name, pass_, k, "next"))
        for s in slots:
            st.close(s)
    assert any(key[3] for key in st.prompt_graphs), "no chunk of several sequences was recorded"
    assert replayed > 0
    st.ops.raise_on_kernel_error()
    st.cache.check_consistent()
