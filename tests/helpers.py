"""Shared by the tests: model folders with random weights, the plain implementation's
logits for a folder, and error measures."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import torch

from tests.plain import minicpm4_plain as plain

# Largest allowed |engine - plain| relative to the largest |plain logit| of the compared rows.
# float32: both sides are fp32 with different summation orders.  bfloat16: weights are the
# same bf16 values on both sides; activations and the cache are rounded to bf16 in the engine.
TOL = {"float32": 5e-6, "bfloat16": 1.5e-2}


def make_folder(cfgd: dict, out_dir: str, seed: int, dtype: str, std: float = 0.02, norm_mean: float = 1.0) -> str:
    from cpmcu_b200.models.model import Model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import write_model_folder

    arch = architecture(cfgd["architectures"][0])
    cfg = arch.config_class.from_dict(cfgd)
    specs = Model(arch.model_spec(cfg), None).weight_specs()
    tdtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    return write_model_folder(cfg, specs, out_dir, seed, tdtype, std, norm_mean)


def read_folder(folder: str):
    """(raw config dictionary, tensors by name) read without the package under test."""
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    # cloned: the reader's tensors are views of the file, which a test may rewrite
    return cfg, {k: v.clone() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


_plain_cache: Dict[tuple, torch.Tensor] = {}


def plain_logits(folder: str, ids: Sequence[int], schedule=None) -> torch.Tensor:
    key = (folder, tuple(ids), None if schedule is None else tuple(schedule))
    if key not in _plain_cache:
        cfg, w = read_folder(folder)
        _plain_cache[key] = plain.forward(cfg, w, list(ids), schedule=schedule)
    return _plain_cache[key]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    log = os.environ.get("CPMCU_TEST_ERRLOG")
    if log:
        with open(log, "a") as f:
            f.write(f"{os.environ.get('PYTEST_CURRENT_TEST', '?')} {err:.3e}\n")
    return err


def random_ids(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def firm_positions(folder: str, ids: Sequence[int], min_gap: float = 0.002) -> torch.Tensor:
    """Positions whose block choice (sparse attention) is firm in the plain implementation: the gap
    between the last chosen and the first rejected block score is at least ``min_gap`` (relative) in
    every layer and kv head.  Elsewhere a rounding of the scores may choose another block, which is
    no fault of an engine that computes in bfloat16; tests leave such positions out.  With random
    weights the block scores of a query lie close together (most gaps are below one percent), so
    the bound is set just above the rounding of bfloat16 scores, not at a comfortable distance."""
    cfg, w = read_folder(folder)
    margins = [float("inf")] * len(ids)
    plain.forward(cfg, w, list(ids), margins=margins)
    return torch.tensor([m >= min_gap for m in margins])


_firm_cache: Dict[tuple, torch.Tensor] = {}


def check_rows(got: torch.Tensor, folder: str, ids: Sequence[int], positions: Sequence[int], dtype: str, label=None) -> float:
    """Asserts that ``got`` (one row of logits per entry of ``positions``) agrees with the plain
    implementation's logits of the sequence ``ids`` at these positions.  In bfloat16, for a folder
    with sparse attention, positions whose block choice is a near tie are left out (firm_positions)."""
    want = plain_logits(folder, ids)
    positions = list(positions)
    keep = torch.ones(len(positions), dtype=torch.bool)
    cfg, _ = read_folder(folder) if dtype == "bfloat16" else ({}, None)
    if cfg.get("sparse_config"):
        key = (folder, tuple(ids))
        if key not in _firm_cache:
            _firm_cache[key] = firm_positions(folder, ids)
        keep = _firm_cache[key][torch.tensor(positions)]
        if not bool(keep.any()):
            return 0.0                                          # nothing but near ties among these rows
    err = rel_err(got[keep], want[torch.tensor(positions)][keep])
    assert err < TOL[dtype], (label, dtype, err)
    return err
