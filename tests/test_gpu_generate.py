"""Generation through the Python entry point and the command line, against the plain
implementation generating greedily token by token."""
import os
import subprocess
import sys

import pytest
import torch

from tests import configs, helpers
from tests.plain import minicpm4_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_greedy(folder, prompt, n_new, stop=()):
    cfg, w = helpers.read_folder(folder)
    ids, out, rows = list(prompt), [], []
    for _ in range(n_new):
        logits = plain.forward(cfg, w, ids)[-1]
        tok = plain.sample_token(logits, 0.0, 0.0)
        rows.append(logits)
        out.append(tok)
        ids.append(tok)
        if tok in stop:
            break
    return out, rows


def check_greedy(folder, prompt, got, dtype, n_new, stop=()):
    """fp32: the very tokens of the plain implementation.  bf16: every chosen token is within the rounding margin of
    the plain implementation's best logit, given the engine's own history; that is a check of the loop, not of the
    values: the logits of the decode runner are compared row by row in test_gpu_runner.py."""
    if dtype == "float32":
        want, _ = plain_greedy(folder, prompt, n_new, stop)
        assert got == want
        return
    cfg, w = helpers.read_folder(folder)
    ids = list(prompt)
    for tok in got:
        logits = plain.forward(cfg, w, ids)[-1]
        margin = helpers.TOL["bfloat16"] * float(logits.abs().max())
        assert float(logits[tok]) >= float(logits.max()) - 2 * margin, (len(ids), tok)
        ids.append(tok)


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_batch_tiny_a(model_folders, dtype, graph):
    """Tiny A's workload: batch 3 with prompts of 5/17/33 tokens, 16 greedy steps."""
    from cpmcu_b200 import LLM

    folder = model_folders("tiny_a", configs.tiny_a(), 0, dtype)
    llm = LLM(folder, dtype=dtype, cuda_graph=graph, max_tokens=64 * 16, chunk_length=64)
    prompts = [helpers.random_ids(512, n, 7 + n) for n in (5, 17, 33)]
    res = llm.generate_batch(prompts, generation_length=16)
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 16 and r.reason == "length"
        check_greedy(folder, p, r.tokens, dtype, 16)
    # the same requests one at a time give the same tokens
    if dtype == "float32":
        for p, r in zip(prompts, res):
            toks, _, _ = llm.generate(p, generation_length=16)
            assert toks == r.tokens
    llm.cache.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_b_sampling_batch(model_folders, dtype):
    """Tiny B's workload: batch 4 with prompts of 1/40/97/150 tokens, 24 steps at temperature
    0.8 with a fixed seed.  A sequence's draws do not depend on its batch: each request run
    alone gives the same tokens."""
    from cpmcu_b200 import LLM

    folder = model_folders("tiny_b", configs.tiny_b(), 1, dtype)
    prompts = [helpers.random_ids(1000, n, 3 + n) for n in (1, 40, 97, 150)]
    llm = LLM(folder, dtype=dtype, cuda_graph=True, temperature=0.8, random_seed=11, max_tokens=64 * 24)
    res = llm.generate_batch(prompts, generation_length=24)
    again = llm.generate_batch(prompts, generation_length=24)
    assert [r.tokens for r in res] == [r.tokens for r in again]
    assert all(len(r.tokens) == 24 for r in res)
    if dtype == "float32":
        # every drawn token is what the plain implementation draws from its own logits with the same random number
        cfg, w = helpers.read_folder(folder)
        for i in (0, 2):
            ids = list(prompts[i])
            for n, tok in enumerate(res[i].tokens[:6]):
                logits = plain.forward(cfg, w, ids)[-1]
                u = plain.philox_uniform(11, i, n)
                wts = plain.sampling_weights(logits, 0.8)
                c = torch.cumsum(wts, 0)
                lo = float(c[tok - 1]) if tok > 0 else 0.0
                slack = 1e-4 * float(c[-1])
                assert lo - slack <= u * float(c[-1]) <= float(c[tok]) + slack
                ids.append(tok)


def test_stop_tokens_and_lengths(model_folders):
    from cpmcu_b200 import LLM

    folder = model_folders("tiny_a", configs.tiny_a(), 0, "float32")
    llm = LLM(folder, dtype="float32", cuda_graph=True, max_tokens=64 * 8, max_batch=2)
    prompts = [helpers.random_ids(512, n, 70 + n) for n in (9, 30, 4, 12, 21)]
    free = llm.generate_batch(prompts, generation_length=12)
    stop = free[1].tokens[3]
    res = llm.generate_batch(prompts, generation_length=12, terminators=[stop])
    for p, r, f in zip(prompts, res, free):
        if stop in f.tokens:
            cut = f.tokens.index(stop) + 1
            assert r.tokens == f.tokens[:cut] and r.reason == "stop"      # the stop token is kept
        else:
            assert r.tokens == f.tokens and r.reason == "length"
    assert llm.last_stats.batches == 3                                      # five requests, two at a time
    llm.cache.check_consistent()
    assert llm.cache.slots.n_held == 1                                      # only the decode runner's scratch sequence


def test_stream_and_cli(model_folders):
    from cpmcu_b200 import LLM

    folder = model_folders("tiny_c", configs.tiny_c(), 5, "bfloat16")
    llm = LLM(folder, max_tokens=64 * 4)
    prompt = helpers.random_ids(777, 11, 1)
    toks, decode_time, prefill_time = llm.generate(prompt, generation_length=8)
    items = list(llm.generate(prompt, generation_length=8, use_stream=True))
    assert [it["token"] for it in items] == toks
    assert items[-1]["is_finished"] and not items[0]["is_finished"]
    out = subprocess.run([sys.executable, "-m", "cpmcu_b200.cli", "--model-path", folder, "--prompt-ids",
                          ",".join(map(str, prompt)), "--num-generate", "8", "--use-stream", "false",
                          "--max-tokens", "256"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip() == "[0] " + " ".join(map(str, toks))


def test_cli_random_weights_mode_and_dense_switch(tmp_path):
    """The command line's random-weights mode writes a model folder from a config.json and a seed and generates
    from it; with --dense the configuration's sparse attention is left out, and the tokens are those of the
    plain implementation on the same folder with the sparse_config taken away."""
    import json

    cfgd = configs.tiny_b()
    cfg_path, folder = str(tmp_path / "config.json"), str(tmp_path / "model")
    with open(cfg_path, "w") as f:
        json.dump(cfgd, f)
    prompt = helpers.random_ids(cfgd["vocab_size"], 150, 4)              # longer than dense_len: sparse would differ
    out = subprocess.run([sys.executable, "-m", "cpmcu_b200.cli", "--random-weights", "9", "--config", cfg_path,
                          "--model-path", folder, "--dtype", "float32", "--dense", "true", "--prompt-ids",
                          ",".join(map(str, prompt)), "--num-generate", "5", "--use-stream", "false", "--ignore-eos", "true",
                          "--max-tokens", "512"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    got = [int(x) for x in out.stdout.strip().split("] ")[1].split()]
    cfg, w = helpers.read_folder(folder)
    cfg = dict(cfg)
    cfg.pop("sparse_config", None)
    ids = list(prompt)
    for tok in got:
        assert tok == plain.sample_token(plain.forward(cfg, w, ids)[-1], 0.0, 0.0)
        ids.append(tok)


def test_trace_run_program(model_folders, tmp_path):
    """bin/trace_run end to end: two requests start together, the shorter ends first."""
    import json
    import numpy as np

    folder = model_folders("tiny_a", configs.tiny_a(), 0, "float32")
    a, b = helpers.random_ids(512, 40, 1), helpers.random_ids(512, 75, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [29, 0]},
                                     {"id": "b", "tokens": b[:70], "want": []}], "end": []}]
    for t in range(10):
        entries = [{"id": "a", "tokens": [a[30 + t]], "want": [0]}]
        if t < 5:
            entries.append({"id": "b", "tokens": [b[70 + t]], "want": [0]})
        steps.append({"step": t + 1, "entries": entries, "end": (["b"] if t == 4 else []) + (["a"] if t == 9 else [])})
    out_dir = tmp_path / "out"
    env = dict(os.environ)
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out_dir), "--max-tokens", "256"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stderr
    assert p.stdout.split() == [x for s in steps for x in ("done", str(s["step"]))]
    wa, wb = helpers.plain_logits(folder, a), helpers.plain_logits(folder, b)
    got0 = torch.from_numpy(np.fromfile(out_dir / "0.f32", dtype="<f4").reshape(2, 512))
    assert helpers.rel_err(got0, wa[[29, 0]]) < helpers.TOL["float32"]
    for t in range(10):
        got = torch.from_numpy(np.fromfile(out_dir / f"{t + 1}.f32", dtype="<f4").reshape(-1, 512))
        want = [wa[30 + t]] + ([wb[70 + t]] if t < 5 else [])
        assert helpers.rel_err(got, torch.stack(want)) < helpers.TOL["float32"]


@pytest.mark.parametrize("name,make,dtype", [("tiny_b", configs.tiny_b, "bfloat16"), ("tiny_a", configs.tiny_a, "float32")])
def test_many_random_batches_leave_the_cache_clean(model_folders, name, make, dtype):
    """Forty batches of random sizes (more prompts than the batch limit, lengths from 1 to 300, stop tokens, greedy
    and temperature, one to thirty new tokens): every result obeys its stop rule, no slot or page is lost, and
    greedy float32 tokens are those of the plain implementation."""
    import random

    from cpmcu_b200 import LLM

    cfgd = make()
    folder = model_folders(name, cfgd, 0, dtype)
    llm = LLM(folder, dtype=dtype, cuda_graph=True, max_tokens=64 * 160, max_batch=16, chunk_length=64)
    cfg, w = helpers.read_folder(folder)
    rng = random.Random(5)
    vocab = cfgd["vocab_size"]
    for b in range(40):
        n = rng.randint(1, 24)
        prompts = [helpers.random_ids(vocab, rng.choice([1, 2, 5, 17, 63, 64, 65, 100, 130, 300]), rng.randint(0, 10 ** 6))
                   for _ in range(n)]
        gen = rng.choice([1, 2, 7, 30])
        temp = rng.choice([0.0, 0.0, 0.8])
        stops = [rng.randrange(vocab) for _ in range(rng.choice([0, 3, 40]))]
        res = llm.generate_batch(prompts, generation_length=gen, terminators=stops, temperature=temp)
        assert len(res) == n
        for r in res:
            assert 1 <= len(r.tokens) <= gen
            assert all(t not in stops for t in r.tokens[:-1])
            assert len(r.tokens) == gen or r.tokens[-1] in stops
        llm.cache.check_consistent()
        assert llm.cache.slots.n_held == 1                      # only the decode runner's scratch sequence
        if temp == 0.0 and dtype == "float32" and b % 8 == 0:
            i = rng.randrange(n)
            ids = list(prompts[i])
            for tok in res[i].tokens:
                assert tok == plain.sample_token(plain.forward(cfg, w, ids)[-1], 0.0, 0.0), (b, i, len(ids))
                ids.append(tok)
    llm.ops.raise_on_kernel_error()


def test_storage_is_one_arena_with_regions(model_folders):
    """The Python entry point lays weights, step workspace, per-sequence state and key-value pages out in one
    allocation; a memory limit that leaves no room, and a step larger than the workspace was sized for, are refused
    with an error that names the region, before anything runs."""
    from cpmcu_b200 import LLM
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.memory import PoolExhausted

    folder = model_folders("tiny_b", configs.tiny_b(), 1, "bfloat16")
    llm = LLM(folder, dtype="bfloat16", cuda_graph=True, max_tokens=64 * 16, chunk_length=64, max_batch=4)
    llm.init_storage()
    llm.load_from_hf()
    arena = llm.storage.arena
    assert list(arena.regions) == ["weights", "workspace", "frame0", "frame1", "state", "cache"]
    lo, hi = arena.buffer.data_ptr(), arena.buffer.data_ptr() + arena.total
    att = llm.model.blocks[0].mixer
    lane = llm.cache.lane(0)
    for t in (att.w_qkv, att.w_o, llm.model.embedding.weight, lane.k, lane.v, lane.pooled, lane.page_table):
        assert lo <= t.data_ptr() < hi
    prompts = [helpers.random_ids(1000, n, n) for n in (70, 9, 130)]
    res = llm.generate_batch(prompts, generation_length=8)
    assert all(len(r.tokens) == 8 for r in res)
    ws = llm.storage.workspace
    assert 0 < ws.peaks()[1] <= ws.frames[0].size and ws.peaks()[0] <= ws.persistent.size
    # the same tokens as with torch's allocator
    plain_llm = LLM(folder, dtype="bfloat16", cuda_graph=True, max_tokens=64 * 16, chunk_length=64, max_batch=4, use_arena=False)
    assert [r.tokens for r in plain_llm.generate_batch(prompts, generation_length=8)] == [r.tokens for r in res]
    # a step of more sequences than the workspace was sized for
    slots = llm.stepper.open(5)
    with pytest.raises(PoolExhausted, match="region 'workspace'.*sequences"):
        llm.step([SequenceStep(s, [1, 2, 3], [2]) for s in slots])
    for s in slots:
        llm.stepper.close(s)
    # a chunk larger than the workspace was sized for
    llm.stepper.chunk_tokens = 512
    slot = llm.stepper.open(1)[0]
    with pytest.raises(PoolExhausted, match="region 'workspace'.*tokens"):
        llm.step([SequenceStep(slot, helpers.random_ids(1000, 300, 1), [299])])
    llm.stepper.close(slot)
    # a memory limit that leaves nothing
    tight = LLM(folder, dtype="bfloat16", memory_limit=1e-6)
    with pytest.raises(PoolExhausted, match="memory_limit"):
        tight.init_storage()
    assert isinstance(PoolExhausted("cache", 1, 0), MemoryError)
