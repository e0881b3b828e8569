"""A whole architecture that the package does not know, defined by the tests: a typed
configuration, three parts of its own, a model specification and one registration.

    layer 0: attention with a position encoding that is not a rotation and has a learned tensor of its own,
             then a feed-forward that routes every token to one of several experts;
    layer 1: a mixer with state of its own (a decaying sum per sequence, kept in the cache's per-sequence
             state and updated on the device through the step's slot indices), then a gated feed-forward;
    layer 2: the package's attention with rotary positions, then a gated feed-forward.

Importing this module registers everything (``--plugin tests.toy_arch`` on the command line,
``CPMCU_PLUGINS=tests.toy_arch`` elsewhere); no file of the package is changed.  It is no model
of anyone's: the parts are the simplest that exercise the interfaces.  ``plain_logits`` is its
plain implementation (whole sequence, no cache), written with the functions of tests/plain.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Dict, List, Sequence

import torch

from cpmcu_b200.config.base import ConfigError
from cpmcu_b200.parts import (FEED_FORWARDS, MIXERS, POSITIONS, CacheNeeds, FeedForward, LayerSpec, Mixer, ModelSpec,
                              PartSpec, PositionEncoding, ScheduleEntry, WeightSpec)
from cpmcu_b200.registry import Architecture, register_architecture

NAME = "ToyStateForCausalLM"


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    inner_size: int
    state_size: int
    decay: float
    n_experts: int
    expert_size: int
    wave_amplitude: float
    eps: float
    residual_scale: float
    rope_theta: float = 10000.0
    eos_token_id: int = -1
    architecture: str = NAME

    @classmethod
    def from_dict(cls, data: dict) -> "ToyConfig":
        fields = {f for f in cls.__dataclass_fields__ if f != "architecture"}
        missing = sorted(f for f in fields - {"rope_theta", "eos_token_id"} if f not in data)
        if missing:
            raise ConfigError(f"config.json: required keys missing: {missing}")
        cfg = cls(**{k: data[k] for k in fields if k in data})
        if cfg.n_heads % cfg.n_kv_heads:
            raise ConfigError("config.json: n_heads must be a multiple of n_kv_heads")
        return cfg

    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [NAME]
        return d


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------

def _dev(ops):
    return ops.device if ops is not None else "cpu"


@POSITIONS.register("toy_wave_learned")
class LearnedWave(PositionEncoding):
    """q and k times (1 + amplitude * cos(position * rate_c)) per dimension c, with ``rate`` a tensor of the
    checkpoint: not a rotation of pairs, and an encoding with weights of its own."""

    def __init__(self, ops, head_dim: int, amplitude: float):
        super().__init__(ops)
        self.d, self.amplitude = int(head_dim), float(amplitude)
        self.rate = None

    def weight_specs(self):
        return {"rate": WeightSpec((self.d,), "vector")}

    def load_weights(self, tensors):
        self.rate = tensors["rate"].float()

    def apply(self, ctx, q, k):
        f = 1.0 + self.amplitude * torch.cos(ctx.positions.float()[:, None] * self.rate[None, :])
        q.mul_(f[:, None, :].to(q.dtype))
        k.mul_(f[:, None, :].to(k.dtype))


@MIXERS.register("toy_decay_state")
class DecayState(Mixer):
    """s_t = decay * s_{t-1} + W_in y_t;  out_t = W_out s_t, s one fp32 vector per sequence in the cache's
    per-sequence state.  A prompt is walked on the host's description of the batch; a decode step (one token per
    sequence) is done with device indices only, so that it can be recorded into a graph."""

    def __init__(self, ops, hidden_size: int, state_size: int, decay: float):
        super().__init__(ops)
        self.h, self.n, self.decay = int(hidden_size), int(state_size), float(decay)

    def weight_specs(self):
        return {"in.weight": WeightSpec((self.n, self.h)), "out.weight": WeightSpec((self.h, self.n))}

    def load_weights(self, tensors):
        self.w_in, self.w_out = tensors["in.weight"].float(), tensors["out.weight"].float()

    def cache_needs(self):
        return CacheNeeds(state={"s": ((self.n,), torch.float32)})

    def forward(self, ctx, y, lane, writes_cache):
        state = lane.state["s"]
        if ctx.is_decode:
            idx = ctx.slot_dev.long()
            s = self.decay * state.index_select(0, idx) + y.float() @ self.w_in.T
            state.index_copy_(0, idx, s)          # padding entries all write the scratch slot: harmless
            return (s @ self.w_out.T).to(y.dtype)
        out = torch.empty_like(y)
        o = 0
        for slot, n in zip(ctx.slots, ctx.q_lens):
            s = state[slot].clone()
            u = y[o:o + n].float() @ self.w_in.T
            for t in range(n):
                s = self.decay * s + u[t]
                out[o + t] = (self.w_out @ s).to(y.dtype)
            state[slot] = s
            o += n
        return out


@FEED_FORWARDS.register("toy_routed_dense")
class RoutedExperts(FeedForward):
    """out = p_e * W2_e relu(W1_e y) for the expert e with the largest router logit, p = softmax of the router
    logits in 32-bit.  Every expert is computed for every token and the others are masked out: slow, but with
    shapes that do not depend on the data, so the step can be recorded."""

    def __init__(self, ops, hidden_size: int, expert_size: int, n_experts: int):
        super().__init__(ops)
        self.h, self.m, self.e = int(hidden_size), int(expert_size), int(n_experts)

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
        out = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
        for e in range(self.e):
            hid = torch.relu(self.ops.linear(y, self.w1[e]))
            gate = torch.where(choice == e, p[:, e], torch.zeros_like(p[:, e]))
            out += self.ops.linear(hid, self.w2[e]).float() * gate[:, None]
        return out.to(y.dtype)


NAMES = {"mixer_norm": "n1.", "mixer": "mix.", "feed_forward_norm": "n2.", "feed_forward": "ff."}


def model_spec(c: ToyConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"hidden_size": c.hidden_size, "eps": c.eps})
    att = {"hidden_size": c.hidden_size, "n_heads": c.n_heads, "n_kv_heads": c.n_kv_heads, "head_dim": c.head_dim}
    wave = PartSpec("gqa_attention", dict(att, position_name="pos.", position=PartSpec(
        "toy_wave_learned", {"head_dim": c.head_dim, "amplitude": c.wave_amplitude})))
    rope = PartSpec("gqa_attention", dict(att, position=PartSpec("rope", {"head_dim": c.head_dim, "theta": c.rope_theta})))
    decay = PartSpec("toy_decay_state", {"hidden_size": c.hidden_size, "state_size": c.state_size, "decay": c.decay})
    routed = PartSpec("toy_routed_dense", {"hidden_size": c.hidden_size, "expert_size": c.expert_size,
                                           "n_experts": c.n_experts})
    gated = PartSpec("gated_ffn", {"hidden_size": c.hidden_size, "intermediate_size": c.inner_size})
    block = PartSpec("pre_norm_residual", {"residual_scale": c.residual_scale})
    layers = [LayerSpec(block, wave, routed, norm, norm, "L0.", NAMES),
              LayerSpec(block, decay, gated, norm, norm, "L1.", NAMES),
              LayerSpec(block, rope, gated, norm, norm, "L2.", NAMES)]
    return ModelSpec(NAME, c.hidden_size, c.vocab_size,
                     PartSpec("scaled_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "scale": 2.0}),
                     layers, [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2)], norm,
                     PartSpec("scaled_lm_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "scale": 1.0}),
                     embedding_name="emb.", final_norm_name="fn.", head_name="head.",
                     stop_token_ids=(c.eos_token_id,) if c.eos_token_id >= 0 else (), max_positions=4096)


register_architecture(Architecture(name=NAME, config_class=ToyConfig, model_spec=model_spec))


def config_dict() -> dict:
    return {"architectures": [NAME], "vocab_size": 210, "hidden_size": 48, "n_heads": 3, "n_kv_heads": 1, "head_dim": 16,
            "inner_size": 56, "state_size": 20, "decay": 0.85, "n_experts": 3, "expert_size": 40, "wave_amplitude": 0.3,
            "eps": 1e-5, "residual_scale": 0.7}


# ---------------------------------------------------------------------------
# plain implementation
# ---------------------------------------------------------------------------

def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int]):
    """(logits [S, vocab], per position the gap between the two best router logits)."""
    from tests.plain import minicpm4_plain as plain

    w = {k: v.float().cpu() for k, v in weights.items()}
    H, heads, kv, d = cfg["hidden_size"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    E, M, eps, rs = cfg["n_experts"], cfg["expert_size"], cfg["eps"], cfg["residual_scale"]
    S = len(ids)
    pos = torch.arange(S, dtype=torch.float32)
    x = plain.embed(list(ids), w["emb.weight"], 2.0)
    # layer 0
    y = plain.rms_norm(x, w["L0.n1.weight"], eps)
    f = 1.0 + cfg["wave_amplitude"] * torch.cos(pos[:, None] * w["L0.mix.pos.rate"][None, :])
    q = (y @ w["L0.mix.q_proj.weight"].T).view(S, heads, d) * f[:, None, :]
    k = (y @ w["L0.mix.k_proj.weight"].T).view(S, kv, d) * f[:, None, :]
    v = (y @ w["L0.mix.v_proj.weight"].T).view(S, kv, d)
    x = x + rs * (plain.dense_attention(q, k, v, 1 / math.sqrt(d)).reshape(S, -1) @ w["L0.mix.o_proj.weight"].T)
    y = plain.rms_norm(x, w["L0.n2.weight"], eps)
    logits = y @ w["L0.ff.router.weight"].T
    top = logits.topk(2, dim=-1).values
    margin = top[:, 0] - top[:, 1]
    prob = torch.softmax(logits, dim=-1)
    out = torch.zeros_like(y)
    for t in range(S):
        e = int(logits[t].argmax())
        out[t] = prob[t, e] * (w["L0.ff.w2"].view(E, H, M)[e] @ torch.relu(w["L0.ff.w1"].view(E, M, H)[e] @ y[t]))
    x = x + rs * out
    # layer 1
    y = plain.rms_norm(x, w["L1.n1.weight"], eps)
    s = torch.zeros(cfg["state_size"])
    a = torch.empty_like(y)
    for t in range(S):
        s = cfg["decay"] * s + w["L1.mix.in.weight"] @ y[t]
        a[t] = w["L1.mix.out.weight"] @ s
    x = x + rs * a
    y = plain.rms_norm(x, w["L1.n2.weight"], eps)
    x = x + rs * plain.gated_ffn(y, {"f." + n: w["L1.ff." + n] for n in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")}, "f.")
    # layer 2
    acfg = {"num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": d, "hidden_size": H,
            "rope_theta": cfg.get("rope_theta", 10000.0), "max_position_embeddings": 4096}
    y = plain.rms_norm(x, w["L2.n1.weight"], eps)
    a, _ = plain.attention_layer(y, w, "L2.mix.", acfg, torch.arange(S))
    x = x + rs * a
    y = plain.rms_norm(x, w["L2.n2.weight"], eps)
    x = x + rs * plain.gated_ffn(y, {"f." + n: w["L2.ff." + n] for n in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")}, "f.")
    return plain.lm_head(plain.rms_norm(x, w["fn.weight"], eps), {"lm_head.weight": w["head.weight"]}, {}, 1.0), margin


def plain_greedy(cfg: dict, weights, prompt: Sequence[int], n_new: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n_new):
        logits, _ = plain_logits(cfg, weights, ids)
        tok = int((logits[-1] == logits[-1].max()).nonzero()[0])
        out.append(tok)
        ids.append(tok)
    return out
