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
# folder -> [rows kept, rows seen] among the rows of bf16 comparisons that lie beyond the folder's dense_len
sparse_rows_seen: Dict[str, List[int]] = {}
# Smallest share of such rows that must survive the near-tie filter.  Measured with the plain implementation on
# random sequences of 150 to 400 tokens: tiny B (three layers, one block chosen per layer) keeps 26 to 29 % at the
# configuration's std of 0.02 and about 50 % at 0.08 (single stretches of 32 positions keep as little as 6 %); tiny D
# at std 0.08 keeps every row up to 250 tokens and 53 % at 400.  This filter is only the fallback for steps that
# leave no record of their block choices; a run whose fallback comparisons keep less than the floor compares too
# little to count.
SPARSE_KEEP_FLOOR = 0.15


# Largest amount by which a block an engine chose in bfloat16 may score below the plain rule's cut-off (relative):
# the rounding of bf16 queries moves a block score by a few parts in a thousand.
SELECT_SLACK = 1e-2


def record_blocks(stepper) -> None:
    """From now on the stepper's sparse attention parts leave their block choices in ``stepper.taps``."""
    stepper.taps = {"block_lists": []}


def taken_blocks(stepper, slot: int) -> Dict[int, Dict[int, List[List[int]]]]:
    """The block choices recorded for the sequence in ``slot`` (cache lane -> position -> one ascending list per
    kv head; a query that saw at most dense_len keys has none), removed from the record so that the slot's next
    sequence starts empty."""
    out: Dict[int, Dict[int, List[List[int]]]] = {}
    rest = []
    for lane, slots, token_seq, positions, lists in stepper.taps["block_lists"]:
        seq_of, pos, rows = token_seq.tolist(), positions.tolist(), lists.cpu()
        mine = [t for t, j in enumerate(seq_of) if slots[j] == slot]
        for t in mine:
            per_head = []
            for h in range(rows.shape[1]):
                row = rows[t, h].tolist()
                if row[0] == -2:                                            # "dense": not a choice
                    per_head = None
                    break
                per_head.append(row[:next((x for x, b in enumerate(row) if b < 0), len(row))])
            if per_head is not None:
                out.setdefault(lane, {})[pos[t]] = per_head
        if len(mine) < len(seq_of):
            rest.append((lane, slots, token_seq, positions, lists))
    stepper.taps["block_lists"] = rest
    return out


def check_rows(got: torch.Tensor, folder: str, ids: Sequence[int], positions: Sequence[int], dtype: str, label=None,
               blocks=None) -> float:
    """Asserts that ``got`` (one row of logits per entry of ``positions``) agrees with the plain
    implementation's logits of the sequence ``ids`` at these positions.

    bfloat16 and sparse attention: a choice between two blocks of nearly equal score may fall the other way
    in an engine that rounds its queries to bf16.  With ``blocks`` (the engine's own choices for this sequence,
    see ``taken_blocks``) every row is compared: the plain implementation attends to the blocks the engine chose,
    and each choice must be the plain rule's up to SELECT_SLACK.  Without ``blocks`` (a step that was recorded
    into a graph leaves no record) positions whose plain choice is a near tie in some layer are left out
    (firm_positions); how many rows that leaves is counted in ``sparse_rows_seen`` and checked against
    SPARSE_KEEP_FLOOR over all calls by ``check_sparse_rows_kept``."""
    positions = list(positions)
    cfg, w = read_folder(folder) if dtype == "bfloat16" else ({}, None)
    if cfg.get("sparse_config") and blocks is not None:
        slack: List[float] = []
        want = plain.forward(cfg, w, list(ids), chosen={lane: blocks.get(lane, {}) for lane in range(cfg["num_hidden_layers"])},
                             slack=slack)
        assert max(slack, default=0.0) < SELECT_SLACK, (label, "a chosen block scores below the rule's cut-off", max(slack))
        err = rel_err(got, want[torch.tensor(positions)])
        assert err < TOL[dtype], (label, dtype, err)
        return err
    want = plain_logits(folder, ids)
    keep = torch.ones(len(positions), dtype=torch.bool)
    if cfg.get("sparse_config"):
        key = (folder, tuple(ids))
        if key not in _firm_cache:
            _firm_cache[key] = firm_positions(folder, ids)
        keep = _firm_cache[key][torch.tensor(positions)]
        beyond = torch.tensor([p + 1 > cfg["sparse_config"].get("dense_len", 0) for p in positions])
        seen = sparse_rows_seen.setdefault(folder, [0, 0])
        seen[0] += int((keep & beyond).sum())
        seen[1] += int(beyond.sum())
        if not bool(keep.any()):
            return float("nan")                                 # nothing but near ties among these rows; counted above
    err = rel_err(got[keep], want[torch.tensor(positions)][keep])
    assert err < TOL[dtype], (label, dtype, err)
    return err


def check_sparse_rows_kept() -> None:
    """Over all bf16 comparisons of a run: of the rows beyond dense_len, at least SPARSE_KEEP_FLOOR were compared."""
    for folder, (kept, total) in sparse_rows_seen.items():
        if total >= 40:
            assert kept >= SPARSE_KEEP_FLOOR * total, (folder, "rows compared", kept, "of", total)


def runner_parity(stepper, seqs: Sequence[Sequence[int]], prompt_lens: Sequence[int], check, use_graph: bool,
                  seed: int = 0) -> int:
    """Drives the decode runner (the way into the model that generation uses) with given tokens and checks the logits
    of every step.  ``seqs[i]`` is a whole sequence of token ids; its first ``prompt_lens[i]`` tokens go through the
    step function as the prompt, the others are fed to the runner one per step, so sequences leave the batch at
    different steps and the runner is restarted on the ones that stay (smaller buckets, padding entries).
    When a sequence ends, ``check(i, rows, positions, blocks)`` is called with its fp32 logits at ``positions`` (the
    prompt's last position and every decoded one) and the block choices recorded for it (None unless
    ``record_blocks`` was called on the stepper and the steps ran without a graph).  Returns the number of decode
    steps."""
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.engine.decode import DecodeRunner
    from cpmcu_b200.sampling import SamplingParams

    n = len(seqs)
    slots = stepper.open(n)
    out = stepper.step([SequenceStep(s, list(ids[:L]), [L - 1]) for s, ids, L in zip(slots, seqs, prompt_lens)])
    rows = [[out[i:i + 1].clone()] for i in range(n)]
    places = [[prompt_lens[i] - 1] for i in range(n)]

    def done(i):
        blocks = taken_blocks(stepper, slots[i]) if stepper.taps is not None and not use_graph else None
        check(i, torch.cat(rows[i]), places[i], blocks)
        stepper.close(slots[i])

    runner = DecodeRunner(stepper, use_graph=use_graph, seed=seed)
    at = list(prompt_lens)                          # index of the next token to feed, per sequence
    live = [i for i in range(n) if at[i] < len(seqs[i])]
    for i in range(n):
        if i not in live:
            done(i)
    changed, steps = True, 0
    while live:
        feed = [seqs[i][at[i]] for i in live]
        if changed:
            runner.start([slots[i] for i in live], feed, live, [0] * len(live), [SamplingParams()] * len(live))
        else:
            runner.feed(feed)
        runner.step()
        out = runner.logits().clone()
        steps += 1
        still = []
        for r, i in enumerate(live):
            rows[i].append(out[r:r + 1])
            places[i].append(at[i])
            at[i] += 1
            if at[i] < len(seqs[i]):
                still.append(i)
            else:
                done(i)
        changed = len(still) != len(live)
        live = still
    stepper.close(runner.pad_slot)
    return steps
