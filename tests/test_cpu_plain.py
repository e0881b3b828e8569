"""The plain implementation checked against itself: identities that hold whatever the
weights are, so a slip in one of its functions shows without any other implementation."""
import math

import pytest
import torch

from tests import configs, helpers
from tests.plain import minicpm4_plain as plain


@pytest.fixture(scope="module")
def folder_b(tmp_path_factory):
    return helpers.make_folder(configs.tiny_b(), str(tmp_path_factory.mktemp("b")), 1, "float32")


def test_scale_folding_identity(folder_b):
    """scripts/model_convert/minicpm2llama.py:28-39: folding the three scales into the weights
    gives the same logits."""
    cfg, w = helpers.read_folder(folder_b)
    ids = helpers.random_ids(1000, 90, 0)
    a = plain.forward(cfg, w, ids, dtype=torch.float64)
    cfg2, w2 = plain.fold_scales(cfg, w)
    b = plain.forward(cfg2, w2, ids, dtype=torch.float64)
    assert float((a - b).abs().max()) < 1e-12


def test_causality_and_float32_accuracy(folder_b):
    cfg, w = helpers.read_folder(folder_b)
    ids = helpers.random_ids(1000, 120, 1)
    full = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:77])[-1], full[76], atol=1e-6)
    assert helpers.rel_err(full, plain.forward(cfg, w, ids, dtype=torch.float64)) < 5e-6


def test_sparse_rules(folder_b):
    cfg, w = helpers.read_folder(folder_b)
    ids = helpers.random_ids(1000, 150, 2)
    sparse = plain.forward(cfg, w, ids)
    dense_cfg = dict(cfg, sparse_config=None)
    dense = plain.forward(dense_cfg, w, ids)
    assert torch.equal(sparse[:64], dense[:64])                       # up to dense_len keys: dense
    assert float((sparse[64:] - dense[64:]).abs().max()) > 1e-4       # beyond: blocks are really dropped
    everything = dict(cfg, sparse_config=dict(cfg["sparse_config"], topk=1000))
    assert helpers.rel_err(plain.forward(everything, w, ids), dense) < 1e-6
    # the choice: leading block, local window, and topk - init_blocks others
    sp = cfg["sparse_config"]
    q = torch.randn(150, 4, 32)
    k = torch.randn(150, 1, 32)
    ck = plain.compress_keys(k, sp["kernel_size"], sp["kernel_stride"])
    assert ck.shape[0] == (150 - 8) // 4 + 1
    assert torch.allclose(ck[3, 0], k[12:20, 0].mean(0), atol=1e-6)
    blocks = plain.select_blocks(q[149], ck, 149, 1 / math.sqrt(32), sp)[0]
    assert blocks[0] == 0 and blocks[-2:] == [8, 9] and len(blocks) == 1 + 1 + 2
    assert 1 <= blocks[1] <= 7


def test_rope_table_rules():
    cfg = configs.tiny_b()
    inv, mag = plain.rope_table(cfg)
    assert mag == pytest.approx(math.sqrt(1 + math.log(4) / math.log(64)))
    assert inv[0] == pytest.approx(1.0) and inv[-1] == pytest.approx(1 / (8.0 * 1e6 ** (30 / 32)), rel=1e-5)
    short = dict(cfg, max_position_embeddings=64)
    inv_s, mag_s = plain.rope_table(short)
    assert mag_s == 1.0 and inv_s[-1] == pytest.approx(1 / (1e6 ** (30 / 32)), rel=1e-5)
    # rotation keeps the norm (times the magnitude) and q.k depends on the distance only
    u = torch.randn(1, 1, 32)
    r5 = plain.rotate(u, torch.tensor([5]), inv, 1.0)
    assert float(r5.norm()) == pytest.approx(float(u.norm()), rel=1e-5)
    v = torch.randn(1, 1, 32)
    d1 = (plain.rotate(u, torch.tensor([9]), inv, 1.0) * plain.rotate(v, torch.tensor([4]), inv, 1.0)).sum()
    d2 = (plain.rotate(u, torch.tensor([105]), inv, 1.0) * plain.rotate(v, torch.tensor([100]), inv, 1.0)).sum()
    assert float(d1) == pytest.approx(float(d2), abs=1e-4)


def test_philox_and_sampling():
    # known answer of Philox4x32-10 for a zero key and zero counter (Random123 test vector)
    assert plain.philox_uniform(0, 0, 0) == (0x6627E8D5 >> 8) / 16777216.0
    us = [plain.philox_uniform(7, 3, n) for n in range(2000)]
    assert 0.45 < sum(us) / len(us) < 0.55 and min(us) >= 0 and max(us) < 1
    logits = torch.tensor([0.0, 2.0, 2.0, -1.0])
    assert plain.sample_token(logits, 0.0, 0.3) == 1                    # tie: lowest index
    w = plain.sampling_weights(logits, 1.0, top_p=0.5)
    assert w[0] == 0 and w[3] == 0 and w[1] > 0 and w[2] > 0            # ties at the threshold are kept together
    assert plain.sample_token(logits, 1.0, 0.999) == 3 and plain.sample_token(logits, 1.0, 0.0) == 0
