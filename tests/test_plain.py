"""The plain implementation against mxxm-t/llmx's own CPU code, and its sampler against definitions.

tests/golden/*.npz hold logits the reference's float32 CPU path gave for tiny random models
(made by tests/golden/make_golden.py, which writes the weights with this repository's
random-weights mode from the same seeds).  The plain implementation must agree with them within
the reference's own float32 bound for such a comparison (2e-5 on logits, tests/common.py:458).
"""
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from configs import TINY_A, TINY_B

HERE = os.path.dirname(os.path.abspath(__file__))


def _weights(raw, seed):
    from llmx_b200.config import Qwen3Config
    from llmx_b200.registry import architecture_of
    from llmx_b200.weights import RandomSource
    cfg = Qwen3Config.from_dict(raw)
    model = architecture_of(cfg.to_dict()).build(cfg)
    src = RandomSource(model.tensor_specs(), seed, dtype=torch.float32, skip_optional=True)
    return {n: src.tensor(n).numpy() for n in src.names()}


@pytest.mark.parametrize("tag,raw", [("tiny_a", TINY_A), ("tiny_b", TINY_B)])
def test_plain_matches_reference_cpu_code(tag, raw):
    g = np.load(os.path.join(HERE, "golden", f"{tag}.npz"))
    w = _weights(raw, int(g["seed"]))
    logits = plain.forward(raw, w, g["ids"].tolist())
    assert logits.shape == g["whole"].shape
    assert np.abs(logits - g["whole"]).max() <= 2e-5
    assert np.abs(logits - g["steps"]).max() <= 2e-5


def test_plain_matches_the_reference_s_hugging_face_golden():
    """The second anchor, independent of the reference's own code: float32 logits Hugging Face's Qwen3 gave for a
    model of odd sizes (width 37, head width 42, vocabulary 257), tied and untied (tests/hf_anchor.py)."""
    import hf_anchor
    fixtures = hf_anchor.fixtures()
    if fixtures is None:
        pytest.skip("the golden file is not at hand")
    assert {tied for tied, *_ in fixtures} == {True, False}
    for tied, cfg, w, cases in fixtures:
        for ids, want in cases:
            got = plain.forward(cfg, w, ids)
            assert np.abs(got[-1] - want).max() <= hf_anchor.BOUND, (tied, len(ids))


def test_rms_norm_and_rope_by_hand():
    x = np.array([[3.0, 4.0]], dtype=np.float32)
    w = np.array([2.0, 0.5], dtype=np.float32)
    y = plain.rms_norm(x, w, 0.0)
    r = 1.0 / np.sqrt(12.5)
    assert np.allclose(y, [[3 * r * 2, 4 * r * 0.5]], atol=1e-6)
    cos, sin = plain.rope_tables(3, 4, 10000.0)
    assert np.allclose(cos[0], 1) and np.allclose(sin[0], 0)
    assert np.isclose(cos[2, 0], np.cos(2.0), atol=1e-6) and np.isclose(sin[2, 1], np.sin(2 * 0.01), atol=1e-7)
    v = np.array([[[1.0, 2.0, 3.0, 4.0]]], dtype=np.float32)
    out = plain.rope_rotate(v, cos[1:2], sin[1:2])
    c0, s0, c1, s1 = cos[1, 0], sin[1, 0], cos[1, 1], sin[1, 1]
    assert np.allclose(out[0, 0], [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1], atol=1e-6)


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((6, 4, 8)).astype(np.float32)
    k = rng.standard_normal((6, 2, 8)).astype(np.float32)
    v = rng.standard_normal((6, 2, 8)).astype(np.float32)
    o = plain.attention(q, k, v)
    assert np.allclose(o[0, 0], v[0, 0], atol=1e-6) and np.allclose(o[0, 3], v[0, 1], atol=1e-6)
    k2, v2 = k.copy(), v.copy()
    k2[5], v2[5] = 100.0, 100.0                         # a later key changes no earlier row
    assert np.allclose(plain.attention(q, k2, v2)[:5], o[:5])
    ow = plain.attention(q, k, v, window=1)             # a window of one key: the row's own value
    assert np.allclose(ow[:, 0], v[:, 0], atol=1e-6)


def test_sampler_definitions():
    logits = np.array([1.0, 3.0, 3.0, -1.0, 2.0], dtype=np.float32)
    assert plain.sample(logits, 0.0, 0, 1.0, 0.0, 0.5) == 1                      # greedy, ties to the lowest id
    assert plain.sample(logits, 0.0, 0, 1.0, 0.0, 0.5, masked=1) == 2
    assert plain.sample(logits, 1.0, 1, 1.0, 0.0, 0.999) == 1                    # top-k of one is the best
    assert plain.sample(logits, 1.0, 0, 1.0, 1.0, 0.7) in (1, 2)                 # min_p 1 keeps the likeliest
    # temperature: the draw walks id order; weights are e^-2, 1, 1, e^-4, e^-1
    w = np.exp(np.array([-2, 0, 0, -4, -1.0]))
    cum = np.cumsum(w) / w.sum()
    for r in (0.01, 0.3, 0.6, 0.85, 0.999):
        assert plain.sample(logits, 1.0, 0, 1.0, 0.0, r) == int(np.searchsorted(cum, r, side="right"))
    # top-p walks rank order: 1, 2, 4, 0, 3
    assert plain.sample(logits, 1.0, 0, 0.5, 0.0, 0.99) in (1, 2)
    assert plain.sample(logits, 1.0, 0, 0.9, 0.0, 0.99) == 4
    # penalties: a seen token's positive logit is divided, then presence and frequency come off
    assert plain.sample(logits, 0.0, 0, 1.0, 0.0, 0.5, penalty=2.0, gen=[1]) == 2
    assert plain.sample(logits, 0.0, 0, 1.0, 0.0, 0.5, presence=0.5, frequency=0.3, gen=[1, 2, 2]) == 1
    rng = plain.XorShift64()
    assert rng.next() == ((lambda x: x)(rng.s)) and 0.0 <= rng.unit() < 1.0
