"""A plain, slow implementation of dense Qwen3: whole sequences, no cache, one function per part.

Written from the reference's formulas (each function cites file:line in
mxxm-t/llmx) in numpy float32.  It shares no code with `llmx_b200`: it reads the
model folder with the `safetensors` library and config.json with `json`, and is
what every engine test compares against.  `tests/golden/` holds logits of the
reference's own CPU code for a tiny random model; `tests/test_plain.py` checks
this file against them once.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import numpy as np

F = np.float32


def load_folder(model_dir: str):
    """(config dict, {name: float32 array}) of a model folder."""
    import torch
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = load_file(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: v.to(torch.float32).numpy() for k, v in tensors.items()}


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (nearest even) and widen back: what a bfloat16 path stores."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=F)).to(torch.bfloat16).to(torch.float32).numpy()


# ---------------------------------------------------------------------------
def embedding(table: np.ndarray, ids) -> np.ndarray:
    """x[r, :] = W_E[ids[r], :]   (src/model/arch/blocks.hpp:95-97; src/backends/cpu/cpu_backend.hpp:233-257)."""
    return table[np.asarray(ids, dtype=np.int64)].astype(F)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """s = sum x_i^2; r = 1 / sqrt(s / n + eps); y_i = x_i * (r * w_i)
    (src/backends/cpu/cpu_backend.hpp:1437-1459)."""
    x = x.astype(F)
    n = x.shape[-1]
    s = np.sum(x * x, axis=-1, keepdims=True, dtype=F)
    r = (F(1.0) / np.sqrt(s / F(n) + F(eps))).astype(F)
    return (x * (r * w.astype(F))).astype(F)


def rope_frequencies(head_dim: int, theta: float, yarn: Optional[dict] = None) -> np.ndarray:
    """freq_i = powf(theta, -2 i / D) (src/model/rope.hpp:25-28); under YaRN the blend of the
    interpolated and the plain frequency along the ramp (src/model/rope.hpp:159-188, float32 branch)."""
    half = head_dim // 2
    i = np.arange(half, dtype=F)
    if yarn is None:
        return np.power(F(theta), F(-2.0) * i / F(head_dim)).astype(F)
    factor, original = float(yarn["factor"]), int(yarn["original_max_position_embeddings"])
    beta_fast, beta_slow = float(yarn.get("beta_fast", 32.0)), float(yarn.get("beta_slow", 1.0))

    def correction(rot):
        return head_dim * math.log(original / (rot * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(correction(beta_fast)), 0.0)
    high = min(math.ceil(correction(beta_slow)), float(head_dim - 1))
    if low == high:
        high += 0.001
    out = np.zeros(half, dtype=F)
    for k in range(half):
        power = F(np.power(F(theta), F(2 * k) / F(head_dim)))
        extra = F(1.0) / power
        inter = F(1.0) / (F(factor) * power)
        ramp = min(max((F(k) - F(low)) / F(high - low), F(0.0)), F(1.0))
        extrapolate = F(1.0) - F(ramp)
        out[k] = inter * (F(1.0) - extrapolate) + extra * extrapolate
    return out


def rope_tables(positions: int, head_dim: int, theta: float, yarn: Optional[dict] = None):
    """cos/sin[pos, i] = cosf/sinf((float) pos * freq_i), times 0.1 ln(factor) + 1 under YaRN
    (src/model/rope.hpp:191-217, attention factor :145)."""
    freq = rope_frequencies(head_dim, theta, yarn)
    pos = np.arange(positions, dtype=F)[:, None]
    angle = (pos * freq[None, :]).astype(F)
    cos, sin = np.cos(angle).astype(F), np.sin(angle).astype(F)
    if yarn is not None:
        scale = F(0.1 * math.log(float(yarn["factor"])) + 1.0)
        cos, sin = (cos * scale).astype(F), (sin * scale).astype(F)
    return cos, sin


def rope_rotate(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotate-half over the whole head: a = x[i], b = x[i + D/2];
    x[i] = a cos_i - b sin_i; x[i + D/2] = a sin_i + b cos_i
    (src/backends/cpu/cpu_backend.hpp:1461-1480).  x [T, heads, D]; cos/sin [T, D/2]."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1).astype(F)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: Optional[int] = None,
              scale: Optional[float] = None) -> np.ndarray:
    """Causal grouped-query attention of one whole sequence.
    q [T, H, D], k/v [T, G, D]; query head h reads kv head h // (H / G); the row at position p
    attends t in [lo, p]; s_t = dot(q, k_t) * scale, scale = 1 / sqrt(D); softmax; o = sum p_t v_t
    (src/backends/cpu/cpu_backend.hpp:980-1029)."""
    T, H, D = q.shape
    G = k.shape[1]
    ratio = H // G
    scale = F(1.0 / math.sqrt(D)) if scale is None else F(scale)
    out = np.zeros((T, H, D), dtype=F)
    for h in range(H):
        g = h // ratio
        s = (q[:, h, :] @ k[:, g, :].T).astype(F) * scale          # [T, T]
        for p in range(T):
            lo = 0 if window is None else max(0, p - window + 1)
            row = s[p, lo:p + 1]
            e = np.exp(row - row.max()).astype(F)
            prob = (e / e.sum(dtype=F)).astype(F)
            out[p, h, :] = prob @ v[lo:p + 1, g, :]
    return out


def silu(g: np.ndarray) -> np.ndarray:
    """silu(g) = g / (1 + exp(-g))   (src/backends/cpu/cpu_backend.hpp:1677)."""
    return (g / (F(1.0) + np.exp(-g))).astype(F)


def swiglu_ffn(h: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray, act_round=None) -> np.ndarray:
    """down(silu(gate h) * up h)   (src/model/arch/blocks.hpp:101-106)."""
    g, u = (h @ w_gate.T).astype(F), (h @ w_up.T).astype(F)
    a = (silu(g) * u).astype(F)
    if act_round is not None:
        a = act_round(a)
    return (a @ w_down.T).astype(F)


def attention_block(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, cfg: dict, cos, sin, act_round=None,
                    window: Optional[int] = None, cache_round="same") -> np.ndarray:
    """Projections, per-head q/k RMSNorm before the rotation, attention, output projection
    (src/model/arch/qwen3.hpp:272-295)."""
    H, G = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg["head_dim"]
    T = h.shape[0]
    eps = cfg["rms_norm_eps"]
    q = (h @ w[pre + "q_proj.weight"].T).astype(F).reshape(T, H, D)
    k = (h @ w[pre + "k_proj.weight"].T).astype(F).reshape(T, G, D)
    v = (h @ w[pre + "v_proj.weight"].T).astype(F).reshape(T, G, D)
    q = rope_rotate(rms_norm(q, w[pre + "q_norm.weight"], eps), cos, sin)
    k = rope_rotate(rms_norm(k, w[pre + "k_norm.weight"], eps), cos, sin)
    if cache_round == "same":   # the cache has the path's type unless it is given one of its own
        cache_round = act_round
    if act_round is not None:   # what a reduced-precision path stores: queries ...
        q = act_round(q)
    if cache_round is not None:  # ... and, in the cache, keys and values
        k, v = cache_round(k), cache_round(v)
    o = attention(q, k, v, window=window).reshape(T, H * D)
    if act_round is not None:
        o = act_round(o)
    return (o @ w[pre + "o_proj.weight"].T).astype(F)


def normalized_config(cfg: dict) -> dict:
    """Defaults as the reference reads them (src/model/arch/qwen3.hpp:70-88)."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rms_norm_eps", 1e-6)
    c.setdefault("tie_word_embeddings", False)
    c.setdefault("rope_scaling", None)
    return c


def forward(cfg: dict, w: Dict[str, np.ndarray], ids, act_round=None, cache_round="same") -> np.ndarray:
    """Logits [T, vocab] of one whole sequence: embed, L x (x += attn(norm x); x += ffn(norm x)),
    final norm, head (src/model/passes.hpp:771-830; head src/model/arch/blocks.hpp:267-272).

    `act_round` (optional) rounds what a reduced-precision path rounds: the inputs of every
    matrix product and what the cache stores.  None is the float32 model.  `cache_round`: the rounding of keys and
    values in the cache when the cache has a type of its own ("same": the path's; None: a 32-bit cache).
    """
    cfg = normalized_config(cfg)
    T = len(ids)
    eps = cfg["rms_norm_eps"]
    yarn = cfg["rope_scaling"]
    if yarn is not None:
        yarn = dict(yarn)
        yarn.setdefault("original_max_position_embeddings", cfg.get("max_position_embeddings", 4096))
    cos, sin = rope_tables(T, cfg["head_dim"], cfg["rope_theta"], yarn)
    r = act_round if act_round is not None else (lambda a: a)
    x = embedding(w["model.embed_tokens.weight"], ids)
    for l in range(cfg["num_hidden_layers"]):
        pre = f"model.layers.{l}."
        h = r(rms_norm(x, w[pre + "input_layernorm.weight"], eps))
        x = (x + attention_block(h, w, pre + "self_attn.", cfg, cos, sin, act_round, cache_round=cache_round)).astype(F)
        h = r(rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps))
        x = (x + swiglu_ffn(h, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"],
                            w[pre + "mlp.down_proj.weight"], act_round)).astype(F)
    h = r(rms_norm(x, w["model.norm.weight"], eps))
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return (h @ head.T).astype(F)


# ---------------------------------------------------------------------------
# Sampling, as the reference defines it.
class XorShift64:
    """xorshift64; unit() = (next >> 40) / 2^24   (src/inference/sampler.hpp:21-32)."""

    def __init__(self, seed: int = 0):
        self.s = 0x9E3779B97F4A7C15
        if seed:
            self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next(self) -> int:
        x = self.s
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = x
        return x

    def unit(self) -> float:
        return float(F((self.next() >> 40) * (1.0 / 16777216.0)))


def argmax_lowest(scores: np.ndarray, skip: int = -1) -> int:
    """Largest score, ties to the lowest id, `skip` passed over (src/inference/sampler.hpp:88-132)."""
    best, best_score = -1, None
    for i, s in enumerate(scores):
        if i == skip:
            continue
        if best < 0 or s > best_score:
            best, best_score = i, s
    return best


def sample(logits: np.ndarray, temp: float, top_k: int, top_p: float, min_p: float, r: float,
           penalty: float = 1.0, presence: float = 0.0, frequency: float = 0.0, gen=(), masked: int = -1) -> int:
    """One draw as the reference makes it (src/inference/sampler.hpp:258-378): penalties, greedy at
    temp <= 0, else weights exp((s - best) / temp) over the top-k set, nucleus measured best first,
    min-p cutting the tail; the draw walks id order without top-p and rank order with it."""
    n = len(logits)
    score = np.array(logits, dtype=F)
    skip = masked if (0 <= masked < n and n > 1) else -1
    if gen:
        if penalty > 0 and penalty != 1.0:
            for t in set(gen):
                if t < n:
                    v = F(logits[t])
                    score[t] = v / F(penalty) if v > 0 else v * F(penalty)
        if presence != 0.0 or frequency != 0.0:
            counts: Dict[int, int] = {}
            for t in gen:
                if t < n:
                    counts[t] = counts.get(t, 0) + 1
            for t, c in counts.items():
                score[t] -= F(presence) + F(frequency) * F(c)
    if temp <= 0:
        return argmax_lowest(score, skip)
    ids = [i for i in range(n) if i != skip]
    m = len(ids)
    keep = top_k if (0 < top_k < m) else m
    ranked = sorted(ids, key=lambda i: (-float(score[i]), i))
    kept = sorted(ranked[:keep])
    best = ranked[0]

    def weight(i):
        return float(F(np.exp(F((score[i] - score[best]) / F(temp)))))

    if top_p >= 1.0:
        ws = [weight(i) for i in kept]
        if min_p > 0:
            ws = [0.0 if x < min_p else x for x in ws]
        target = r * sum(ws)
        acc = 0.0
        for i, x in zip(kept, ws):
            acc += x
            if target < acc:
                return i
        return best
    total = sum(weight(i) for i in kept)
    goal = top_p * total
    nucleus, nw = 0, 0.0
    while True:
        nw += weight(ranked[nucleus])
        nucleus += 1
        if not (nucleus < keep and nw < goal):
            break
    if min_p > 0:
        last = nucleus
        while last > 1 and weight(ranked[last - 1]) < min_p:
            last -= 1
        if last < nucleus:
            nucleus = last
            nw = sum(weight(ranked[i]) for i in range(nucleus))
    target = r * nw
    acc = 0.0
    for i in range(nucleus):
        acc += weight(ranked[i])
        if target < acc:
            return ranked[i]
    return best
