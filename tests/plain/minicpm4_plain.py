"""A plain, slow implementation of MiniCPM4 (``MiniCPMForCausalLM``) for the tests.

Whole sequences, no cache, no batching, one function per part, everything in
float32 on the CPU (or float64 with ``dtype=torch.float64``).  It shares no code
with the ``cpmcu_b200`` package: it reads the raw ``config.json`` dictionary and a
dictionary of tensors by checkpoint name.

It is written from the reference's formulas: OpenBMB/CPM.cu has no CPU path (every
operation is a CUDA kernel or a cuBLAS call), so its code cannot run where the tests
are written.  It was compared with the reference's own code once on a GPU, for dense
attention with plain rotary encoding: tests/golden holds the logits the unmodified
reference produced for two tiny random models, with the script that made them, and
tests/test_cpu_golden.py compares this implementation with them at every run.  The
sparse path and LongRoPE rest on the formulas alone.  Each function cites the file and
lines of the reference (paths inside the CPM.cu project) that state its formula.
Where the reference's behaviour is not followed, the docstring says so and why.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

Tensor = torch.Tensor


# ---------------------------------------------------------------------------
# constants derived from config.json
# ---------------------------------------------------------------------------

def head_dim(cfg: dict) -> int:
    """cpmcu/llm.py:62-66: head_dim defaults to hidden_size / num_attention_heads."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def scales(cfg: dict) -> Tuple[float, float, float]:
    """cpmcu/llm.py:67-69: (embedding scale, residual scale, logit scale).

    scale_embed = scale_emb (1 if absent); scale_residual = scale_depth / sqrt(layers)
    (1 if absent); scale_lmhead = dim_model_base / hidden_size (1 if absent).
    """
    se = float(cfg.get("scale_emb", 1.0))
    rs = float(cfg["scale_depth"]) / math.sqrt(cfg["num_hidden_layers"]) if cfg.get("scale_depth") is not None else 1.0
    sl = float(cfg["dim_model_base"]) / cfg["hidden_size"] if cfg.get("dim_model_base") is not None else 1.0
    return se, rs, sl


def rope_table(cfg: dict) -> Tuple[Tensor, float]:
    """(inv_freq float32 [d/2], magnitude factor of cos and sin).

    The reference takes inv_freq from another package's rope functions and drops the
    attention factor they return (cpmcu/llm.py:181-192).  The rule written here is the
    LongRoPE one, fixed per model: factors = long_factor if max_position_embeddings >
    original_max_position_embeddings else short_factor; inv_freq[c] = 1 / (factor[c] *
    theta^(2c/d)); magnitude = sqrt(1 + ln(max/orig) / ln(orig)) when extended, else 1.
    Without rope_scaling: factor 1, magnitude 1.
    """
    d = head_dim(cfg)
    theta = float(cfg.get("rope_theta", 10000.0))
    exponent = torch.arange(0, d, 2, dtype=torch.int64).to(torch.float32) / d
    factor = torch.ones(d // 2, dtype=torch.float32)
    magnitude = 1.0
    rs = cfg.get("rope_scaling")
    if rs:
        orig = int(rs.get("original_max_position_embeddings") or cfg["original_max_position_embeddings"])
        max_pos = int(cfg["max_position_embeddings"])
        if max_pos > orig:
            factor = torch.tensor(rs["long_factor"], dtype=torch.float32)
            magnitude = math.sqrt(1.0 + math.log(max_pos / orig) / math.log(orig))
        else:
            factor = torch.tensor(rs["short_factor"], dtype=torch.float32)
    inv_freq = 1.0 / (factor * (theta ** exponent))
    return inv_freq.to(torch.float32), magnitude


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------

def embed(ids: Sequence[int], table: Tensor, scale: float) -> Tensor:
    """src/model/embedding.cuh:7-20 (row gather) and :49-52 (times scale_emb)."""
    return table[torch.tensor(list(ids), dtype=torch.long)] * scale


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """src/model/norm.cuh:7-51: x * rsqrt(sum(x^2)/dim + eps) * weight (weight as stored)."""
    var = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * torch.rsqrt(var + eps) * weight


def rotate(u: Tensor, positions: Tensor, inv_freq: Tensor, magnitude: float) -> Tensor:
    """src/model/rotary.cuh:6-34: for c < d/2, angle = pos * inv_freq[c] (float32);
    u'[c] = u[c] cos - u[c+d/2] sin; u'[c+d/2] = u[c] sin + u[c+d/2] cos.
    u: [S, heads, d].  cos and sin are multiplied by ``magnitude`` (see rope_table)."""
    half = u.shape[-1] // 2
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # float32 product
    cos = (torch.cos(angle) * magnitude).to(u.dtype)[:, None, :]
    sin = (torch.sin(angle) * magnitude).to(u.dtype)[:, None, :]
    a, b = u[..., :half], u[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def dense_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, window: int = 0) -> Tensor:
    """src/model/attn.cuh:201-226 with the causal rule of src/flash_attn/src/mask.h:185-211:
    score = q.k * rsqrt(d); query i sees keys j <= i; softmax; sum of p*v.
    q: [S, heads, d]; k, v: [S, kv_heads, d]; kv head of q head h is h // group."""
    S, nh, d = q.shape
    group = nh // k.shape[1]
    out = torch.empty_like(q)
    idx = torch.arange(S)
    visible = idx[None, :] <= idx[:, None]
    if window:
        visible &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kh, vh = k[:, h // group], v[:, h // group]
        s = (q[:, h] @ kh.T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ vh
    return out


def compress_keys(k: Tensor, kernel: int, stride: int) -> Tensor:
    """src/model/minicpm4/minicpm4_kvcache.cuh:6-30: compressed key i is the mean of the
    (rotated) keys [stride*i, stride*i + kernel), per kv head.  k: [S, kv, d] -> [n, kv, d],
    n = number of complete windows."""
    S = k.shape[0]
    n = (S - kernel) // stride + 1 if S >= kernel else 0
    if n <= 0:
        return k.new_zeros((0,) + tuple(k.shape[1:]))
    return torch.stack([k[stride * i: stride * i + kernel].mean(dim=0) for i in range(n)])


def select_blocks(q_p: Tensor, ck: Tensor, p: int, scale: float, sparse: dict,
                  margins: Optional[List[float]] = None) -> List[List[int]]:
    """Key blocks a query at position p attends to, per kv head (InfLLM-v2).

    Reference pieces: stage-1 score = softmax of q against the compressed keys, summed
    over the heads of a group (src/model/minicpm4/minicpm4_attn.cuh:119-141,
    src/flash_attn/src/flash_fwd_kernel.h:1770-2265); block score = max over the compressed
    keys that overlap the block, leading blocks forced, blocks of the local window left
    out of the choice (src/model/minicpm4/minicpm4_kvcache.cuh:64-108); top-k with ties to
    the lower index (src/model/topk.cuh:17, 26).

    The reference lets compressed keys and selection see only earlier chunks, so its
    result depends on the chunk length.  Here the rule is per query: compressed key i is
    visible iff its whole window lies at or before p; the blocks of the local window are
    always attended (the reference's local window is narrower in attention than in the
    selection, src/flash_attn/src/flash_blockmask.h:30, which leaves a gap no query sees);
    ``topk`` counts the forced leading blocks; the compress_lse normaliser is not built.
    q_p: [heads, d]; ck: [n_compressed, kv, d] of the whole sequence.  If ``margins`` is given, the
    relative gap between the last block score that was chosen and the first that was not is appended
    for every kv head (infinity when nothing was left out): a small gap means that rounding may
    choose otherwise.
    """
    ks, st, bs = sparse["kernel_size"], sparse["kernel_stride"], sparse["block_size"]
    init_blocks, topk = sparse.get("init_blocks", 1), sparse["topk"]
    local_blocks = sparse["window_size"] // bs
    nh, n_kv = q_p.shape[0], ck.shape[1]
    group = nh // n_kv
    n_vis = (p + 1 - ks) // st + 1 if p + 1 >= ks else 0
    qb = p // bs
    last_choice = qb - local_blocks            # blocks k <= last_choice can be chosen
    per_block = bs // st
    reach_back = ks // st - 1
    result: List[List[int]] = []
    for j in range(n_kv):
        score = torch.zeros(n_vis, dtype=q_p.dtype)
        if n_vis > 0:
            for h in range(j * group, (j + 1) * group):
                s = (ck[:n_vis, j] @ q_p[h]) * scale
                score += torch.softmax(s, dim=0)
        chosen = set(k for k in range(min(init_blocks, qb + 1)))
        candidates = []
        for k in range(init_blocks, last_choice + 1):
            lo, hi = max(0, k * per_block - reach_back), min(n_vis, (k + 1) * per_block)
            if hi > lo:
                candidates.append((-float(score[lo:hi].max()), k))
        candidates.sort()
        room = max(0, topk - init_blocks)
        chosen.update(k for _, k in candidates[:room])
        if margins is not None:
            if 0 < room < len(candidates):
                last_in, first_out = -candidates[room - 1][0], -candidates[room][0]
                margins.append((last_in - first_out) / max(abs(last_in), 1e-30))
            else:
                margins.append(float("inf"))
        chosen.update(k for k in range(max(0, last_choice + 1), qb + 1))
        result.append(sorted(chosen))
    return result


def selection_slack(q_p: Tensor, ck: Tensor, p: int, scale: float, sparse: dict, lists: List[List[int]]) -> float:
    """How far a given choice of blocks (one ascending list per kv head, as an engine made it) is from the
    rule of ``select_blocks``: 0 if it is the plain choice or differs from it only among equal scores; else the
    largest relative amount by which a chosen block's score lies below the score of the last block the plain rule
    takes (a choice between nearly equal scores that rounding turned the other way gives a tiny number).  The
    forced leading blocks and the blocks of the local window must be exactly those of the rule, and the number
    of chosen blocks too: infinity otherwise."""
    ks, st, bs = sparse["kernel_size"], sparse["kernel_stride"], sparse["block_size"]
    init_blocks, topk = sparse.get("init_blocks", 1), sparse["topk"]
    local_blocks = sparse["window_size"] // bs
    nh, n_kv = q_p.shape[0], ck.shape[1]
    group = nh // n_kv
    n_vis = (p + 1 - ks) // st + 1 if p + 1 >= ks else 0
    qb = p // bs
    last_choice = qb - local_blocks
    per_block, reach_back = bs // st, ks // st - 1
    worst = 0.0
    for j in range(n_kv):
        score = torch.zeros(n_vis, dtype=q_p.dtype)
        if n_vis > 0:
            for h in range(j * group, (j + 1) * group):
                score += torch.softmax((ck[:n_vis, j] @ q_p[h]) * scale, dim=0)
        forced = set(range(min(init_blocks, qb + 1))) | set(range(max(0, last_choice + 1), qb + 1))
        cand = {}
        for k in range(init_blocks, last_choice + 1):
            lo, hi = max(0, k * per_block - reach_back), min(n_vis, (k + 1) * per_block)
            if hi > lo:
                cand[k] = float(score[lo:hi].max())
        room = min(max(0, topk - init_blocks), len(cand))
        got = set(lists[j])
        far = got - forced
        if not forced <= got or len(far) != room or not far <= set(cand):
            return float("inf")
        if room == 0 or room == len(cand):
            continue
        cutoff = sorted(cand.values(), reverse=True)[room - 1]
        for k in far:
            worst = max(worst, (cutoff - cand[k]) / max(abs(cutoff), 1e-30))
    return worst


def sparse_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, sparse: dict,
                     margins: Optional[List[float]] = None, chosen: Optional[Dict[int, List[List[int]]]] = None,
                     slack: Optional[List[float]] = None) -> Tensor:
    """Per query: dense if it sees at most dense_len keys (the reference's sparse_switch,
    src/model/minicpm4/minicpm4_attn.cuh:116), else attention over the keys of its
    selected blocks that are at or before it (src/flash_attn/src/flash_blockmask.h:15-93).
    ``chosen`` (position -> one block list per kv head) replaces the selection for the positions beyond
    dense_len; it must then name every such position."""
    S, nh, d = q.shape
    n_kv = k.shape[1]
    group = nh // n_kv
    bs = sparse["block_size"]
    ck = compress_keys(k, sparse["kernel_size"], sparse["kernel_stride"])
    dense = dense_attention(q, k, v, scale)
    out = dense.clone()
    for p in range(S):
        if p + 1 <= sparse.get("dense_len", 0):
            continue
        here: Optional[List[float]] = [] if margins is not None else None
        if chosen is not None:
            # the blocks an engine chose for this query: attended as given; how far the choice is from the
            # rule goes into ``slack`` (see selection_slack)
            blocks = chosen[p]
            if slack is not None:
                slack.append(selection_slack(q[p], ck, p, scale, sparse, blocks))
        else:
            blocks = select_blocks(q[p], ck, p, scale, sparse, here)
        if margins is not None and chosen is None:
            margins[p] = min(margins[p], min(here))
        for h in range(nh):
            keys = [j for b in blocks[h // group] for j in range(b * bs, min((b + 1) * bs, p + 1))]
            idx = torch.tensor(keys, dtype=torch.long)
            s = (k[idx, h // group] @ q[p, h]) * scale
            out[p, h] = torch.softmax(s, dim=0) @ v[idx, h // group]
    return out


def attention_layer(y: Tensor, w: Dict[str, Tensor], prefix: str, cfg: dict, positions: Tensor,
                    shared_kv: Optional[Tuple[Tensor, Tensor]] = None,
                    margins: Optional[List[float]] = None, chosen=None, slack=None) -> Tuple[Tensor, Tuple[Tensor, Tensor]]:
    """src/model/attn.cuh:185-229: q, k, v projections without bias, rotary on q and k (keys
    are kept rotated), attention, output projection.  Returns (output, (k, v))."""
    nh, nkv, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim(cfg)
    S = y.shape[0]
    inv_freq, magnitude = rope_table(cfg)
    q = (y @ w[prefix + "q_proj.weight"].T).view(S, nh, d)
    q = rotate(q, positions, inv_freq, magnitude)
    if shared_kv is None:
        k = (y @ w[prefix + "k_proj.weight"].T).view(S, nkv, d)
        v = (y @ w[prefix + "v_proj.weight"].T).view(S, nkv, d)
        k = rotate(k, positions, inv_freq, magnitude)
    else:
        k, v = shared_kv
    scale = 1.0 / math.sqrt(d)
    sparse = cfg.get("sparse_config")
    o = sparse_attention(q, k, v, scale, sparse, margins, chosen, slack) if sparse else dense_attention(q, k, v, scale)
    return o.reshape(S, nh * d) @ w[prefix + "o_proj.weight"].T, (k, v)


def gated_ffn(y: Tensor, w: Dict[str, Tensor], prefix: str) -> Tensor:
    """src/model/ffn.cuh:38-50, 77-84 and src/model/activation.cuh:6-18:
    down( gate * sigmoid(gate) * up ), sigmoid(z) = 1 / (1 + exp(-z))."""
    g = y @ w[prefix + "gate_proj.weight"].T
    u = y @ w[prefix + "up_proj.weight"].T
    return (g * (1.0 / (1.0 + torch.exp(-g))) * u) @ w[prefix + "down_proj.weight"].T


def lm_head(y: Tensor, w: Dict[str, Tensor], cfg: dict, scale: float) -> Tensor:
    """src/model/linear.cuh:86-104: logits = (y * scale) @ W^T; a tied head uses the
    embedding matrix (cpmcu/llm.py:136-137)."""
    W = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return (y * scale) @ W.T


# ---------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------

def forward(cfg: dict, weights: Dict[str, Tensor], ids: Sequence[int], dtype: torch.dtype = torch.float32,
            schedule: Optional[Sequence[Tuple[int, int, bool]]] = None,
            margins: Optional[List[float]] = None, chosen: Optional[Dict[int, Dict[int, List[List[int]]]]] = None,
            slack: Optional[List[float]] = None) -> Tensor:
    """Logits [S, vocab] at every position of one sequence.

    Order of operations as src/model/model.cuh:145-153 and src/model/layer.cuh:47-67:
    x = embed * scale_emb; per layer x += rs * attn(norm(x)); x += rs * ffn(norm(x));
    logits = head(norm(x)).  ``schedule`` lists runs (layer, cache lane, writes): a run
    that does not write uses the keys and values an earlier run stored in that lane.
    ``margins``, if given, must be a list of len(ids) infinities; it receives, per position, the
    smallest block-choice gap over all layers and kv heads (see select_blocks).  ``chosen`` (cache lane ->
    position -> block lists) makes the sparse attention use an engine's block choice instead of its own, and
    ``slack`` receives how far each such choice is from the rule (see selection_slack).
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    se, rs, sl = scales(cfg)
    eps = float(cfg["rms_norm_eps"])
    S = len(ids)
    positions = torch.arange(S)
    x = embed(ids, w["model.embed_tokens.weight"], se)
    if schedule is None:
        schedule = [(i, i, True) for i in range(cfg["num_hidden_layers"])]
    lanes: Dict[int, Tuple[Tensor, Tensor]] = {}
    for layer, lane, writes in schedule:
        p = f"model.layers.{layer}."
        y = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        a, kv = attention_layer(y, w, p + "self_attn.", cfg, positions, None if writes else lanes[lane], margins,
                                None if chosen is None else chosen[lane], slack)
        if writes:
            lanes[lane] = kv
        x = x + rs * a
        y = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + rs * gated_ffn(y, w, p + "mlp.")
    y = rms_norm(x, w["model.norm.weight"], eps)
    return lm_head(y, w, cfg, sl)


def fold_scales(cfg: dict, weights: Dict[str, Tensor]) -> Tuple[dict, Dict[str, Tensor]]:
    """scripts/model_convert/minicpm2llama.py:28-39: the same function with the three
    scales folded into the weights (embedding * scale_emb, lm_head * logit scale,
    o_proj and down_proj * residual scale) and the scales set to 1."""
    se, rs, sl = scales(cfg)
    out = {k: v.clone().to(torch.float64) for k, v in weights.items()}
    out["model.embed_tokens.weight"] = out["model.embed_tokens.weight"] * se
    head = (weights["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else weights["lm_head.weight"])
    out["lm_head.weight"] = head.to(torch.float64) * sl
    for i in range(cfg["num_hidden_layers"]):
        for n in (f"model.layers.{i}.self_attn.o_proj.weight", f"model.layers.{i}.mlp.down_proj.weight"):
            out[n] = out[n] * rs
    cfg2 = dict(cfg)
    cfg2.pop("scale_emb", None)
    cfg2.pop("scale_depth", None)
    cfg2.pop("dim_model_base", None)
    cfg2["tie_word_embeddings"] = False
    return cfg2, out


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

def philox_uniform(seed: int, a: int, b: int) -> float:
    """Philox4x32-10 with key = the 64-bit seed and counter (a, b, 0, 0); the first
    output word's top 24 bits as a number in [0, 1)."""
    M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c = [a & mask, b & mask, 0, 0]
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k1) & mask, p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return (c[0] >> 8) / 16777216.0


def sampling_weights(logits: Tensor, temperature: float, top_p: float = 1.0) -> Tensor:
    """cpmcu/llm.py:282-285: softmax(logits / temperature), unnormalised, in float64.
    With top_p < 1, entries below the largest threshold whose kept mass still reaches
    top_p of the total are dropped (the reference has no top-p)."""
    z = logits.to(torch.float64)
    w = torch.exp((z - z.max()) / temperature)
    if top_p < 1.0:
        order = torch.sort(w, descending=True).values
        need = top_p * w.sum()
        csum = torch.cumsum(order, dim=0)
        n_keep = int((csum < need).sum().item()) + 1
        threshold = order[min(n_keep, len(order)) - 1]
        w = torch.where(w >= threshold, w, torch.zeros_like(w))
    return w


def sample_token(logits: Tensor, temperature: float, u: float, top_p: float = 1.0) -> int:
    """Greedy (lowest index on ties) when temperature is 0; else the first index whose
    cumulative weight, in index order, exceeds u * total."""
    if temperature <= 0.0:
        return int((logits == logits.max()).nonzero()[0].item())
    w = sampling_weights(logits, temperature, top_p)
    c = torch.cumsum(w, dim=0)
    return int(min((c > u * c[-1]).nonzero()[0].item(), len(w) - 1))
