"""The decode runner against the plain implementation at the level of logits.

Generation, the command line, the smoke run and the benchmark reach the model through
``DecodeRunner`` (fixed device buffers per bucket, padding entries, optionally a CUDA graph),
not through ``Stepper.step``.  Here the runner is fed the tokens of given sequences and the
logits of every step are compared with the plain implementation's: with and without a graph,
in 32-bit and in bfloat16, with buckets that hold padding entries, a bucket of 64, and batches
that shrink twice as sequences end."""
import pytest
import torch

from tests import configs, helpers

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CONFIGS = {"tiny_a": (configs.tiny_a, 0), "tiny_b": (configs.tiny_b, 1), "tiny_e": (configs.tiny_e, 4)}


def _stepper(folder, dtype, max_tokens, chunk=64, n_slots=None):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.loading import load_model

    _, cfg, model = load_model(folder, dtype)
    cache = Cache(model.cache_needs(), max_tokens, DT[dtype], "cuda:0", n_slots=n_slots, max_step_tokens=chunk)
    return cfg, Stepper(model, cache, chunk_tokens=chunk)


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_e"])
def test_runner_logits_with_padding_and_shrinking_batches(model_folders, name, dtype, graph):
    """Three sequences in a bucket of four (one padding entry); they end after 5, 12 and 20 decode steps, so the
    runner is restarted on two (a full bucket of two) and on one."""
    make, seed = CONFIGS[name]
    folder = model_folders(name, make(), seed, dtype)
    cfg, st = _stepper(folder, dtype, 64 * 16)
    lens, extra = (70, 9, 33), (5, 20, 12)
    seqs = [helpers.random_ids(cfg.vocab_size, L + e, 50 + L) for L, e in zip(lens, extra)]
    helpers.record_blocks(st)                    # eager steps leave their block choices: every sparse row is compared
    rows_seen = []

    def check(i, rows, positions, blocks):
        assert positions == list(range(lens[i] - 1, lens[i] + extra[i]))
        helpers.check_rows(rows, folder, seqs[i], positions, dtype, label=(name, i), blocks=blocks)
        rows_seen.append(len(positions))

    steps = helpers.runner_parity(st, seqs, lens, check, graph)
    assert steps == 20 and sum(rows_seen) == 3 + sum(extra)
    st.cache.check_consistent()
    assert st.cache.tokens_held() == 0


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_runner_logits_bucket_of_64(model_folders, dtype, graph):
    """64 short sequences of tiny A in one bucket; 24 leave after two steps (40 live in a bucket of 64), 20 more
    after four (20 live in a bucket of 32), the rest after six."""
    folder = model_folders("tiny_a", configs.tiny_a(), 0, dtype)
    cfg, st = _stepper(folder, dtype, 64 * 70, n_slots=70)
    lens = [3 + (7 * i) % 38 for i in range(64)]
    extra = [2 if i < 24 else 4 if i < 44 else 6 for i in range(64)]
    seqs = [helpers.random_ids(cfg.vocab_size, L + e, 900 + i) for i, (L, e) in enumerate(zip(lens, extra))]
    count = [0]

    def check(i, rows, positions, blocks):
        helpers.check_rows(rows, folder, seqs[i], positions, dtype, label=i)
        count[0] += len(positions)

    assert helpers.runner_parity(st, seqs, lens, check, graph) == 6
    assert count[0] == 64 + sum(extra)
    st.cache.check_consistent()
