"""The plain implementation's second anchor: logits of a model no code of mxxm-t/llmx computed.

The reference commits `tests/data/baseline_f32.json` (copied here as tests/golden/reference_hf_baseline_f32.json,
data only): float32 logits of Hugging Face's Qwen3ForCausalLM (eager, torch 2.5.1) for a tiny model whose weights
are a pure formula, tied and untied, at sizes that are multiples of nothing -- 2 layers, width 37, feed-forward 19,
2 heads over 1, head width 42, vocabulary 257, theta 10000, eps 1e-6 (tests/f32.py:14-17, tools/gen_baseline.py:954-963).
A case is a text whose token ids are its bytes and the logits at its last position; the reference holds its own
float32 paths to 2e-5 of them (tests/common.py:458).

The weights (tests/f32.py:47-72): one linear congruential stream from 12345, state <- 1664525 state + 1013904223
mod 2^32, value ((state >> 16) & 1023) - 512) / 8192, norm weights 1 + value, drawn tensor by tensor in the
order embedding, final norm, then per layer the four norms (input, post-attention, q, k) and the seven matrices
(q, k, v, o, gate, up, down), then the head if untied; each matrix row-major [out, in].
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
COPY = os.path.join(HERE, "golden", "reference_hf_baseline_f32.json")
ORIGINAL = "/root/reference/tests/data/baseline_f32.json"
BOUND = 2e-5


def config(doc: dict, tied: bool) -> dict:
    c = doc["config"]
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=c["block_count"],
                hidden_size=c["embedding_length"], intermediate_size=c["feed_forward_length"],
                num_attention_heads=c["attention.head_count"], num_key_value_heads=c["attention.head_count_kv"],
                head_dim=c["attention.key_length"], vocab_size=257, rope_theta=10000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=tied, max_position_embeddings=c["context_length"])


def weights(cfg: dict):
    """{HF tensor name: float32 array}, and the sha256 the golden file records for them."""
    E, F, D, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"], cfg["vocab_size"]
    Q, KV = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    state = 12345
    out, digest = {}, hashlib.sha256()

    def draw(name, shape, norm=False):
        nonlocal state
        n = int(np.prod(shape))
        vals = np.empty(n, dtype=np.float64)
        for i in range(n):
            state = (1664525 * state + 1013904223) & 0xFFFFFFFF
            vals[i] = (((state >> 16) & 1023) - 512) / 8192
        if norm:
            vals += 1.0
        arr = vals.astype(np.float32)
        digest.update(arr.astype("<f4").tobytes())
        out[name] = arr.reshape(shape)

    draw("model.embed_tokens.weight", (V, E))
    draw("model.norm.weight", (E,), True)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        draw(p + "input_layernorm.weight", (E,), True)
        draw(p + "post_attention_layernorm.weight", (E,), True)
        draw(p + "self_attn.q_norm.weight", (D,), True)
        draw(p + "self_attn.k_norm.weight", (D,), True)
        draw(p + "self_attn.q_proj.weight", (Q, E))
        draw(p + "self_attn.k_proj.weight", (KV, E))
        draw(p + "self_attn.v_proj.weight", (KV, E))
        draw(p + "self_attn.o_proj.weight", (E, Q))
        draw(p + "mlp.gate_proj.weight", (F, E))
        draw(p + "mlp.up_proj.weight", (F, E))
        draw(p + "mlp.down_proj.weight", (E, F))
    if not cfg["tie_word_embeddings"]:
        draw("lm_head.weight", (V, E))
    return out, digest.hexdigest()


def fixtures():
    """[(tied, config, weights, [(token ids, logits at the last position)])], or None when the golden file is not there."""
    path = ORIGINAL if os.path.exists(ORIGINAL) else COPY
    if not os.path.exists(path):
        return None
    with open(path, encoding="utf-8") as f:
        doc = json.load(f)
    if path == ORIGINAL and os.path.exists(COPY):
        with open(COPY, encoding="utf-8") as f:
            assert json.load(f) == doc, "the copied golden differs from the reference's file"
    out = []
    for fx in doc["fixtures"]:
        cfg = config(doc, fx["tied"])
        w, sha = weights(cfg)
        assert sha == fx["weights_sha256"], "the rebuilt weights are not the golden's"
        cases = [(list(c["text"].encode()), np.asarray(c["logits"], dtype=np.float32)) for c in fx["cases"]]
        out.append((fx["tied"], cfg, w, cases))
    return out
