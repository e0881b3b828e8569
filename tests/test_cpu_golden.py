"""The plain implementation against the reference's own code: logits that the unmodified reference
(OpenBMB/CPM.cu, bfloat16, on a GPU) produced for tiny random models, committed under tests/golden
with the script that made them (tests/golden/make_reference_golden.py), compared here on the CPU
with tests/plain at every run.  Positions: the last token of prompts of several lengths (chunk
edges of the reference's chunked prefill among them) and a dozen tokens decoded one by one."""
import glob
import json
import os

import numpy as np
import pytest
import torch

from tests.golden import make_reference_golden as golden
from tests.plain import minicpm4_plain as plain

FILES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "reference_*.npz")))

# The reference computes in bfloat16 (activations, cache and the returned logits are rounded to it); the plain
# implementation is fp32 on the same bf16 weights.  Largest allowed difference, relative to the largest logit.
TOLERANCE = 2e-2


def test_golden_files_are_there():
    assert len(FILES) >= 2, "tests/golden holds the reference's logits for two tiny models"


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(p) for p in FILES])
def test_plain_implementation_matches_the_reference(path):
    data = np.load(path)
    cfg = json.loads(str(data["config"]))
    cfg["architectures"] = ["MiniCPMForCausalLM"]
    seed = int(data["seed"])
    ids = data["ids"].tolist()
    assert ids == golden.make_tokens(cfg, seed)
    weights = golden.make_weights(cfg, seed)
    logits = plain.forward(cfg, weights, ids)                       # [positions, vocab], whole sequence, no cache
    want = torch.from_numpy(data["logits"])
    got = logits[torch.from_numpy(data["positions"]).long()]
    assert got.shape == want.shape
    scale = float(want.abs().max())
    assert float(want.std()) > 0.05, "logits too flat to tell anything"
    err = float((got - want).abs().max()) / scale
    assert err < TOLERANCE, (os.path.basename(path), err)          # measured: 0.7 % and 1.3 %
    # the largest logit's place agrees wherever the reference's best two are further apart than the tolerance
    top2 = want.topk(2, dim=-1).values
    firm = (top2[:, 0] - top2[:, 1]) > 2 * TOLERANCE * scale
    assert int(firm.sum()) >= len(want) // 3
    assert torch.equal(got.argmax(-1)[firm], want.argmax(-1)[firm])
