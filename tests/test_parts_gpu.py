"""The parts of a layer alone, and an architecture made in this file from the framework's parts plus a
toy mixer with state of its own, registered, built and stepped without a change to the framework.

The toy model exercises what Qwen3 does not: a mixer with fixed-size per-request state, a feed-forward
with a router and experts, a windowed
attention layer whose pages are given back, a partially rotated and an unrotated attention layer, a
block that runs twice (each run with a cache entry of its own), a block that reads the keys
another run of it wrote, and -- all three defined in this file -- a norm that centres and has a bias,
a position encoding that rotates by half the position, and an arrangement in which mixer and
feed-forward read the same normed input.  Its plain implementation below is whole-sequence numpy built from
tests/plain_qwen3.py's functions.
"""
import json
import math
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


# ---------------------------------------------------------------------------------------------
# A toy mixer with state: s_t = decay * s_{t-1} + h_t per request; output s_t W^T.
def _toy_mixer_class():
    from llmx_b200.cache import StateSpec
    from llmx_b200.parts import Part
    from llmx_b200.weights import TensorSpec

    class RunningSumMixer(Part):
        recordable = False          # it walks the batch on the host

        def __init__(self, hidden, decay):
            self.hidden, self.decay = hidden, decay

        def cache_spec(self):
            return StateSpec((self.hidden,), "float32")

        def tensor_specs(self):
            return {"proj.weight": TensorSpec((self.hidden, self.hidden))}

        def load(self, tensors, precision):
            super().load(tensors, precision)
            self.weight = tensors["proj.weight"].float()

        def forward(self, h, step, cache_entry, residual, write_cache=True):
            state = step.state(cache_entry)
            for r in range(step.requests):
                a, n = step.host_row_start[r], step.host_row_count[r]
                slot, slot_out = step.host_state_slots[r], step.host_state_slots_out[r]
                # A request's first token reads a zero state whatever the slot holds.
                s = state[slot].clone() if step.host_history[r] > 0 else torch.zeros(self.hidden, device=h.device)
                outs = []
                for t in range(n):
                    s = self.decay * s + h[a + t].float()
                    outs.append(s)
                state[slot_out] = s          # the request's spare slot: the two swap when the step is committed
                residual[a:a + n] += torch.stack(outs) @ self.weight.T

    return RunningSumMixer


# A toy feed-forward with routing: a float32 router picks one of `experts` small gated MLPs per row.
def _toy_routed_ffn_class():
    from llmx_b200.parts import Part
    from llmx_b200.weights import TensorSpec

    class RoutedFFN(Part):
        recordable = False          # it picks rows on the host side of torch ops

        def __init__(self, hidden, inner, experts):
            self.hidden, self.inner, self.experts = hidden, inner, experts

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.experts, self.hidden))}
            for e in range(self.experts):
                specs[f"experts.{e}.gate_proj.weight"] = TensorSpec((self.inner, self.hidden))
                specs[f"experts.{e}.up_proj.weight"] = TensorSpec((self.inner, self.hidden))
                specs[f"experts.{e}.down_proj.weight"] = TensorSpec((self.hidden, self.inner))
            return specs

        def load(self, tensors, precision):
            super().load(tensors, precision)
            self.w = {n: t.float() for n, t in tensors.items()}

        def forward(self, h, step, residual):
            hf = h.float()
            choice = (hf @ self.w["router.weight"].T).argmax(dim=-1)            # router logits in float32
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                x = hf[rows]
                g, u = x @ self.w[f"experts.{e}.gate_proj.weight"].T, x @ self.w[f"experts.{e}.up_proj.weight"].T
                residual[rows] += (torch.nn.functional.silu(g) * u) @ self.w[f"experts.{e}.down_proj.weight"].T

    return RoutedFFN


# A toy norm (centred, with a bias), a toy position encoding (rotation by half the position) and a toy
# arrangement (mixer and feed-forward side by side on one normed input), with the interfaces the framework's
# own norm, position encoding and block have.
def _toy_extra_classes():
    from llmx_b200.parts import Part
    from llmx_b200.weights import TensorSpec

    class CentredNorm(Part):
        def __init__(self, width, eps):
            self.width, self.eps = width, eps

        def tensor_specs(self):
            return {"weight": TensorSpec((self.width,), "vector", init="one_plus_normal", std=0.05),
                    "bias": TensorSpec((self.width,), "vector", std=0.05)}

        def load(self, tensors, precision):
            super().load(tensors, precision)
            self.weight, self.bias = tensors["weight"].float(), tensors["bias"].float()

        def forward(self, x, out=None, row_index=None, out_dtype=None, zero=None):
            if zero is not None:
                zero.zero_()                         # this norm has no launch of its own to clear it in passing
            if row_index is not None:
                x = x[row_index.long()]
            xf = x.float()
            xc = xf - xf.mean(dim=-1, keepdim=True)
            y = xc * torch.rsqrt((xc * xc).mean(dim=-1, keepdim=True) + self.eps) * self.weight + self.bias
            y = y.to(out_dtype or self.precision.act)
            if out is not None:
                out.copy_(y)
                return out
            return y

    class HalvedPositions(Part):
        """cos/sin tables [positions, rot_dim / 2] of the angles (position / 2) * theta^(-2i / rot_dim)."""

        def __init__(self, head_dim, theta):
            self.rot_dim, self.theta = head_dim, theta
            self.cos = self.sin = None

        def prepare(self, max_positions, device):
            freq = np.power(np.float32(self.theta), np.float32(-2.0) * np.arange(self.rot_dim // 2, dtype=np.float32) / np.float32(self.rot_dim))
            angle = (np.arange(max_positions, dtype=np.float32)[:, None] * np.float32(0.5) * freq[None, :]).astype(np.float32)
            self.cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(device)
            self.sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(device)

    class ParallelBlock(Part):
        """x += mixer(norm(x)) + ffn(norm(x)): one norm, both parts read its output."""

        def __init__(self, norm, mixer, ffn):
            self.norm, self.mixer, self.ffn = norm, mixer, ffn

        def children(self):
            return {"ln": self.norm, "self_attn": self.mixer, "mlp": self.ffn}

        def cache_spec(self):
            return self.mixer.cache_spec()

        def forward(self, x, step, cache_entry, write_cache=True):
            h = self.norm.forward(x)
            self.mixer.forward(h, step, cache_entry, x, write_cache)
            self.ffn.forward(h, step, x)

    return CentredNorm, HalvedPositions, ParallelBlock


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int = 64
    intermediate_size: int = 96
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: int = 16
    vocab_size: int = 128
    window: int = 12
    decay: float = 0.5
    rms_norm_eps: float = 1e-5
    max_position_embeddings: int = 512

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k not in ("architectures", "model_type")})

    def to_dict(self):
        return dict(self.__dict__, architectures=["ToyForCausalLM"], model_type="toy")


def _build_toy(cfg: ToyConfig):
    from llmx_b200.models import LayerStep, Model
    from llmx_b200.parts import (Attention, GatedMLP, LogitsHead, NoPositionEncoding, PreNormBlock, RMSNorm,
                                 RotaryEmbedding, TokenEmbedding)
    E, H, G, D = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    norm = lambda: RMSNorm(E, cfg.rms_norm_eps)   # noqa: E731
    mlp = lambda: GatedMLP(E, cfg.intermediate_size)   # noqa: E731
    blocks = [
        PreNormBlock(norm(), Attention(E, H, G, D, RotaryEmbedding(D, 10000.0, rot_dim=8), qk_norm_eps=cfg.rms_norm_eps),
                     norm(), mlp()),                                                    # 0: partial rotation
        PreNormBlock(norm(), _toy_mixer_class()(E, cfg.decay), norm(),
                     _toy_routed_ffn_class()(E, 48, 3)),                                # 1: state; routed feed-forward
        PreNormBlock(norm(), Attention(E, H, G, D, NoPositionEncoding(), qk_norm_eps=None, window=cfg.window),
                     norm(), mlp()),                                                    # 2: window, no rotation, no q/k norm
    ]
    CentredNorm, HalvedPositions, ParallelBlock = _toy_extra_classes()
    blocks.append(ParallelBlock(CentredNorm(E, cfg.rms_norm_eps),
                                Attention(E, H, G, D, HalvedPositions(D, 10000.0), qk_norm_eps=None),
                                mlp()))                                                 # 3: the file's own norm, encoding, arrangement
    order = [LayerStep(0, 0), LayerStep(1, 1), LayerStep(2, 2), LayerStep(0, 3), LayerStep(2, 2, write_cache=False),
             LayerStep(3, 4)]
    emb = TokenEmbedding(cfg.vocab_size, E)
    head = LogitsHead(norm(), cfg.vocab_size, E, tied_to=emb)
    return Model(embedding=emb, blocks=blocks, head=head, order=order, vocab_size=cfg.vocab_size,
                 max_positions=cfg.max_position_embeddings)


def _plain_toy(cfg: ToyConfig, w, ids):
    """Whole sequence, no cache: the toy model's layer order written out."""
    T, E, H, G, D = len(ids), cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    eps = cfg.rms_norm_eps
    cos, sin = plain.rope_tables(T, 8, 10000.0)
    x = plain.embedding(w["model.embed_tokens.weight"], ids)

    def qkv(h, pre):
        q = (h @ w[pre + "q_proj.weight"].T).reshape(T, H, D)
        k = (h @ w[pre + "k_proj.weight"].T).reshape(T, G, D)
        v = (h @ w[pre + "v_proj.weight"].T).reshape(T, G, D)
        return q, k, v

    def rot8(a):
        out = a.copy()
        out[..., :8] = plain.rope_rotate(a[..., :8], cos, sin)
        return out

    def mlp(x, pre):
        h = plain.rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps)
        return x + plain.swiglu_ffn(h, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"])

    def block0(x):
        pre = "model.layers.0."
        h = plain.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
        q, k, v = qkv(h, pre + "self_attn.")
        q = rot8(plain.rms_norm(q, w[pre + "self_attn.q_norm.weight"], eps))
        k = rot8(plain.rms_norm(k, w[pre + "self_attn.k_norm.weight"], eps))
        o = plain.attention(q, k, v).reshape(T, H * D)
        return mlp(x + o @ w[pre + "self_attn.o_proj.weight"].T, pre)

    def block1(x):
        pre = "model.layers.1."
        h = plain.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
        s, outs = np.zeros(E, dtype=np.float32), []
        for t in range(T):
            s = np.float32(cfg.decay) * s + h[t]
            outs.append(s)
        x = x + np.stack(outs) @ w[pre + "self_attn.proj.weight"].T
        h = plain.rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps)
        choice = (h @ w[pre + "mlp.router.weight"].T).argmax(axis=-1)
        out = x.copy()
        for t in range(T):
            e = int(choice[t])
            out[t] += plain.swiglu_ffn(h[t:t + 1], w[pre + f"mlp.experts.{e}.gate_proj.weight"],
                                       w[pre + f"mlp.experts.{e}.up_proj.weight"], w[pre + f"mlp.experts.{e}.down_proj.weight"])[0]
        return out

    def block2(x, kv=None):
        pre = "model.layers.2."
        h = plain.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
        q, k, v = qkv(h, pre + "self_attn.")
        if kv is not None:
            k, v = kv                                  # the keys and values another run of the block wrote
        o = plain.attention(q, k, v, window=cfg.window).reshape(T, H * D)
        return mlp(x + o @ w[pre + "self_attn.o_proj.weight"].T, pre), (k, v)

    def block3(x):
        pre = "model.layers.3."
        xc = x - x.mean(axis=-1, keepdims=True)
        h = (xc / np.sqrt((xc * xc).mean(axis=-1, keepdims=True) + np.float32(eps)) * w[pre + "ln.weight"] + w[pre + "ln.bias"]).astype(np.float32)
        q, k, v = qkv(h, pre + "self_attn.")
        freq = np.power(np.float32(10000.0), np.float32(-2.0) * np.arange(D // 2, dtype=np.float32) / np.float32(D))
        angle = (np.arange(T, dtype=np.float32)[:, None] * np.float32(0.5) * freq[None, :]).astype(np.float32)
        c, s_ = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
        q, k = plain.rope_rotate(q, c, s_), plain.rope_rotate(k, c, s_)
        o = plain.attention(q, k, v).reshape(T, H * D)
        ffn = plain.swiglu_ffn(h, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"])
        return x + o @ w[pre + "self_attn.o_proj.weight"].T + ffn

    x = block0(x)
    x = block1(x)
    x, kv = block2(x)
    x = block0(x)
    x, _ = block2(x, kv)
    x = block3(x)
    h = plain.rms_norm(x, w["model.norm.weight"], eps)
    return (h @ w["model.embed_tokens.weight"].T).astype(np.float32)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from llmx_b200.registry import register_architecture, unregister_architecture
    from llmx_b200.weights import RandomSource, write_safetensors
    register_architecture(["ToyForCausalLM", "toy"], ToyConfig, _build_toy)
    cfg = ToyConfig()
    d = str(tmp_path_factory.mktemp("toy"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    model = _build_toy(cfg)
    src = RandomSource(model.tensor_specs(), 11, dtype=torch.float32, skip_optional=True)
    tensors = {n: src.tensor(n) * (4.0 if n.endswith("proj.weight") else 1.0) for n in src.names()}
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    yield cfg, d, {n: t.numpy() for n, t in tensors.items()}
    unregister_architecture(["ToyForCausalLM", "toy"])


def test_toy_architecture_is_registered_built_and_stepped(toy):
    """config.json names the toy; the framework builds it from the registry and runs it under every cutting,
    mixed with other requests, with so few pages that they are used again."""
    from llmx_b200.engine import Engine, EngineOptions
    cfg, folder, w = toy
    requests = {f"t{i}": helpers.random_ids(cfg.vocab_size, n, seed=i) for i, n in enumerate([50, 3, 77, 20, 1, 64])}
    refs = {rid: _plain_toy(cfg, w, ids) for rid, ids in requests.items()}
    for make in (helpers.trace_whole, helpers.trace_tail_decoded, helpers.trace_portions, helpers.trace_mixed):
        steps = make(requests)
        engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=helpers.tokens_needed(steps),
                                                       page_size=4, max_requests=4))
        assert len(engine.cache.groups) == 2 and engine.cache.state_entries == [1]      # full and windowed keys; one state
        assert not engine.model.recordable
        got = helpers.run_trace(engine, steps)
        engine.cache.check()
        assert engine.cache.used_pages() == [0, 0] and engine.cache.state_slots.free_slots == 8
        worst = max(float(np.abs(got[(rid, p)] - refs[rid][p]).max()) for rid, ids in requests.items() for p in range(len(ids)))
        scale = max(float(np.abs(r).max()) for r in refs.values())
        assert worst <= 1e-4 * scale, f"{make.__name__}: {worst:.3e} (scale {scale:.3f})"


def test_windowed_group_gives_pages_back_while_the_full_group_keeps_them(toy):
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    cfg, folder, w = toy
    engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=256, page_size=4, max_requests=2))
    ids = helpers.random_ids(cfg.vocab_size, 100, seed=5)
    engine.step([StepEntry("a", ids[:60], [])])
    full = next(i for i, g in enumerate(engine.cache.groups) if g.spec.window is None)
    assert engine.cache.used_pages()[full] == 15 * 2 // 2 and engine.cache.used_pages()[1 - full] <= 4
    for t in ids[60:]:
        engine.step([StepEntry("a", [t], [0])])
        assert engine.cache.used_pages()[1 - full] <= 4
    assert engine.cache.used_pages()[full] == 25


# ---------------------------------------------------------------------------------------------
# Each part of a layer alone, against the plain functions, through the same StepBatch a step builds.
def _single_request_step(n, part, history=0, page=8, kv_heads=2, head_dim=16, dtype=torch.float32, window=None, cache=None):
    """The step of one request that brings `n` rows after `history`, over a cache manager of its own (or `cache`,
    whose request "r" goes on), planned for `part`."""
    from llmx_b200.cache import CacheManager, KVSpec
    from llmx_b200.engine.batch import step_from_requests
    if cache is None:
        cache = CacheManager([KVSpec(kv_heads, head_dim, window)], page, 256, 2, kv_dtype=dtype, device=DEV)
        rc = cache.new_request("r")
        if history:
            rc.prepare(history)
            rc.commit()
    rc = cache.live["r"]
    rc.prepare(n)
    return step_from_requests(cache, [rc], [n], DEV, parts=[part], wants=[(n - 1,)])


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
def test_rmsnorm_part(precision):
    from llmx_b200.parts import Precision, RMSNorm
    part = RMSNorm(96, 1e-5)
    w = torch.rand(96) + 0.5
    part.load({"weight": w.to(DEV)}, Precision.of(precision))
    x = torch.randn(7, 96)
    out = part.forward(x.to(DEV))
    assert out.dtype is Precision.of(precision).act
    ref = plain.rms_norm(x.numpy(), w.numpy(), 1e-5)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= (2 ** -7 if precision == "bfloat16" else 1e-5) * np.abs(ref).max()


def test_rotary_tables_match_the_plain_ones_with_and_without_yarn():
    from llmx_b200.config.qwen3 import YarnScaling
    from llmx_b200.parts import RotaryEmbedding
    for yarn in (None, dict(factor=4.0, original_max_position_embeddings=64, beta_fast=32.0, beta_slow=1.0)):
        part = RotaryEmbedding(32, 1e6, yarn=YarnScaling(**yarn) if yarn else None)
        part.prepare(300, DEV)
        cos, sin = plain.rope_tables(300, 32, 1e6, yarn)
        assert np.abs(part.cos.cpu().numpy() - cos).max() <= 1e-6 and np.abs(part.sin.cpu().numpy() - sin).max() <= 1e-6
    with pytest.raises(ValueError):
        RotaryEmbedding(32, 1e4, rot_dim=34)


@pytest.mark.parametrize("precision,tol", [("float32", 1e-5), ("bfloat16", 2e-2)])
def test_gated_mlp_part(precision, tol):
    from llmx_b200.parts import GatedMLP, Precision
    p = Precision.of(precision)
    E, F = 96, 200
    part = GatedMLP(E, F)
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(s, generator=g) * 0.1).to(p.act) for n, s in
         (("gate_proj.weight", (F, E)), ("up_proj.weight", (F, E)), ("down_proj.weight", (E, F)))}
    part.load({n: t.to(DEV) for n, t in w.items()}, p)
    for rows in (3, 100):          # few rows: separate activation kernel; many rows (bfloat16): the gated product
        h = torch.randn(rows, E, generator=g).to(p.act)
        x = torch.randn(rows, E, generator=g)
        res = x.clone().to(DEV)
        part.forward(h.to(DEV), None, res)
        rnd = plain.round_bf16 if precision == "bfloat16" else None
        ref = x.numpy() + plain.swiglu_ffn(h.float().numpy(), *(w[n].float().numpy() for n in w), act_round=rnd)
        assert np.abs(res.cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("precision,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (6, 2, 64, None), (4, 4, 64, 9)])
def test_attention_part_in_two_portions(precision, tol, heads, kv_heads, head_dim, window):
    """The mixer alone: a first portion fills the cache, a second reads it; together they equal the whole sequence."""
    from llmx_b200.parts import Attention, Precision, RotaryEmbedding
    p = Precision.of(precision)
    E = 64
    part = Attention(E, heads, kv_heads, head_dim, RotaryEmbedding(head_dim, 10000.0), qk_norm_eps=1e-6, window=window)
    g = torch.Generator().manual_seed(1)
    w = {n: (torch.randn(s.shape, generator=g) * (0.2 if s.kind == "matrix" else 0.1) + (0 if s.kind == "matrix" else 1)).to(p.act if s.kind == "matrix" else torch.float32)
         for n, s in part.tensor_specs().items()}
    part.load({n: t.to(DEV) for n, t in w.items()}, p)
    part.prepare(128, DEV)
    T, cut = 37, 21
    h = torch.randn(T, E, generator=g).to(p.act)
    x = torch.zeros(T, E)
    step1 = _single_request_step(cut, part, kv_heads=kv_heads, head_dim=head_dim, dtype=p.act, page=16 if head_dim == 64 else 8, window=window)
    res1 = x[:cut].clone().to(DEV)
    part.forward(h[:cut].to(DEV), step1, 0, res1)
    step1.caches.live["r"].commit()
    step2 = _single_request_step(T - cut, part, cache=step1.caches)
    assert step2.host_history == [cut]
    res2 = x[cut:].clone().to(DEV)
    part.forward(h[cut:].to(DEV), step2, 0, res2)
    got = torch.cat([res1, res2]).cpu().numpy()
    cfg = dict(num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=1e-6)
    cos, sin = plain.rope_tables(T, head_dim, 10000.0)
    wf = {"p." + n: t.float().numpy() for n, t in w.items()}
    ref = plain.attention_block(h.float().numpy(), wf, "p.", cfg, cos, sin,
                                act_round=plain.round_bf16 if precision == "bfloat16" else None, window=window)
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()


def test_embedding_and_tied_head_parts():
    from llmx_b200.parts import LogitsHead, Precision, RMSNorm, TokenEmbedding
    p = Precision.of("float32")
    emb = TokenEmbedding(50, 24)
    table = torch.randn(50, 24)
    emb.load({"weight": table.to(DEV)}, p)
    head = LogitsHead(RMSNorm(24, 1e-6), 50, 24, tied_to=emb)
    head.norm.load({"weight": torch.ones(24, device=DEV)}, p)
    head.load({}, p)
    head.bind_tied()
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32, device=DEV)
    x = emb.forward(ids)
    assert torch.equal(x.cpu(), table[ids.cpu().long()])
    logits = head.forward(x, torch.tensor([3, 1], dtype=torch.int32, device=DEV))
    ref = plain.rms_norm(table[[7, 49]].numpy(), np.ones(24, np.float32), 1e-6) @ table.numpy().T
    assert head.linear.weight.data_ptr() == emb.table.data_ptr()      # tied: the same memory, not a copy
    assert np.abs(logits.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()


def test_layer_order_is_checked():
    from llmx_b200.models import LayerStep, Model
    cfg = ToyConfig()
    m = _build_toy(cfg)
    kw = dict(embedding=m.embedding, blocks=m.blocks, head=m.head, vocab_size=cfg.vocab_size, max_positions=64)
    with pytest.raises(ValueError, match="both write"):
        Model(order=[LayerStep(0, 0), LayerStep(0, 0)], **kw)
    with pytest.raises(ValueError, match="before any step wrote"):
        Model(order=[LayerStep(0, 0, write_cache=False)], **kw)
    with pytest.raises(ValueError, match="needs a cache entry"):
        Model(order=[LayerStep(0, None)], **kw)
    with pytest.raises(ValueError, match="different needs"):
        Model(order=[LayerStep(0, 0), LayerStep(2, 0, write_cache=False)], **kw).cache_entry_specs()
    with pytest.raises(ValueError, match="without gaps"):
        Model(order=[LayerStep(0, 1)], **kw)


def test_a_failed_step_leaves_a_state_mixers_state_as_it_was(toy):
    """State is part of the step's transaction: a step reads a request's state slot and writes its spare, and only a
    commit swaps them.  A step fails on the host after the state mixer of the toy model has run (the step's second
    attention launch comes after it); the same step again gives what a clean engine gives."""
    from llmx_b200 import runtime
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    cfg, folder, w = toy
    ids = helpers.random_ids(cfg.vocab_size, 40, seed=3)
    ref = _plain_toy(cfg, w, ids)
    scale = float(np.abs(ref).max())
    engine = Engine.from_dir(folder, EngineOptions(dtype="float32", kv_tokens=256, page_size=4, max_requests=2))
    engine.step([StepEntry("s", ids[:17], [])])
    slots = (engine.cache.live["s"].state_slot, engine.cache.live["s"].state_slot_out)
    before = engine.cache.state_storage[1].clone()
    runtime.fail_call("llmx_attention_plain", 2)
    with pytest.raises(runtime.KernelError):
        engine.step([StepEntry("s", ids[17:30], [12])])
    runtime.fail_call(None)
    rc = engine.cache.live["s"]
    assert rc.length == 17 and (rc.state_slot, rc.state_slot_out) == slots
    assert torch.equal(engine.cache.state_storage[1][rc.state_slot], before[rc.state_slot])     # the state it will read
    engine.cache.check()
    got = engine.step([StepEntry("s", ids[17:30], [12])]).float().cpu().numpy()[0]
    assert np.abs(got - ref[29]).max() <= 1e-4 * scale
    got = engine.step([StepEntry("s", ids[30:], [9])]).float().cpu().numpy()[0]
    assert np.abs(got - ref[39]).max() <= 1e-4 * scale
    with pytest.raises(RuntimeError, match="fixed-size state"):
        engine.truncate("s", 10)
    engine.end("s")
    assert engine.cache.state_slots.free_slots == 4


# ---------------------------------------------------------------------------------------------
# A mixer of this file that is recordable and plans on the host, and a position encoding with a stream of its own.
def _planned_toy_classes():
    from llmx_b200.parts import Part
    from llmx_b200.parts.base import PartPlan
    from llmx_b200.weights import TensorSpec

    class MeanPlan(PartPlan):
        """The host's share of `HistoryMeanMixer`: for every request 1 / (tokens it holds after the step), as
        fixed-point ints, and the row count of the largest request (a launch decision: in a recorded step it follows
        the recording's shape alone)."""

        def __init__(self, shape):
            self.counts = list(shape.counts)
            self.ints = len(self.counts) + 1
            self.recorded = shape.room > 0
            self.fills = 0

        def fill(self, histories, out):
            self.fills += 1
            out[:len(self.counts)] = [int(round(65536.0 / (h + c))) for h, c in zip(histories, self.counts)]
            out[len(self.counts)] = max(self.counts)

    class HistoryMeanMixer(Part):
        """residual[rows of r] += scale[r] * (h W^T), scale[r] = 1 / (length of r after the step), read on the
        device from the ints its plan put into the step's metadata: tensor ops only, so a step can be recorded."""
        recordable = True
        plans = []

        def __init__(self, hidden):
            self.hidden = hidden

        def cache_spec(self):
            return None

        def tensor_specs(self):
            return {"proj.weight": TensorSpec((self.hidden, self.hidden))}

        def load(self, tensors, precision):
            super().load(tensors, precision)
            self.weight = tensors["proj.weight"].float()

        def plan_step(self, shape):
            plan = MeanPlan(shape)
            HistoryMeanMixer.plans.append(plan)
            return plan

        def forward(self, h, step, cache_entry, residual, write_cache=True):
            ints = step.plan_ints(self)
            assert ints is not None and ints.numel() == step.requests + 1
            scale = ints[:step.requests].float() / 65536.0
            residual += (h.float() @ self.weight.T) * scale[step.row_request.long()][:, None]

    class SecondStreamBias(Part):
        """A feed-forward that adds bias * (the row's position in the step's second position stream)."""
        position_streams = 2

        def __init__(self, hidden):
            self.hidden = hidden

        def tensor_specs(self):
            return {"bias": TensorSpec((self.hidden,), "vector", std=0.05)}

        def load(self, tensors, precision):
            super().load(tensors, precision)
            self.bias = tensors["bias"].float()

        def forward(self, h, step, residual):
            residual += step.position_streams[1].float()[:, None] * self.bias[None, :] * 0.01

    return HistoryMeanMixer, SecondStreamBias


def test_a_recordable_mixer_with_a_plan_of_its_own_and_a_second_position_stream(tmp_path):
    """An architecture of this file whose mixer plans on the host (`plan_step`) and reads its plan's ints on the
    device, and whose feed-forward reads a second position stream the requests bring: registered, built, stepped
    plainly and from recordings, with nothing changed under llmx_b200/engine/ (which knows no part's plan)."""
    from llmx_b200.engine import Engine, EngineOptions, StepEntry
    from llmx_b200.models import LayerStep, Model
    from llmx_b200.parts import LogitsHead, PreNormBlock, RMSNorm, TokenEmbedding
    from llmx_b200.registry import register_architecture, unregister_architecture
    from llmx_b200.weights import RandomSource, write_safetensors
    HistoryMeanMixer, SecondStreamBias = _planned_toy_classes()
    E, V, eps = 48, 90, 1e-5

    @dataclass(frozen=True)
    class Cfg:
        max_position_embeddings: int = 256

        @classmethod
        def from_dict(cls, raw):
            return cls()

        def to_dict(self):
            return dict(architectures=["PlannedToy"], model_type="planned_toy")

    def build(cfg):
        blocks = [PreNormBlock(RMSNorm(E, eps), HistoryMeanMixer(E), RMSNorm(E, eps), SecondStreamBias(E)) for _ in range(2)]
        emb = TokenEmbedding(V, E)
        return Model(embedding=emb, blocks=blocks, head=LogitsHead(RMSNorm(E, eps), V, E, tied_to=emb),
                     order=[LayerStep(0), LayerStep(1), LayerStep(0)], vocab_size=V, max_positions=256)

    register_architecture(["PlannedToy", "planned_toy"], Cfg, build)
    try:
        (tmp_path / "config.json").write_text(json.dumps(Cfg().to_dict()))
        src = RandomSource(build(Cfg()).tensor_specs(), 5, dtype=torch.float32, skip_optional=True)
        tensors = {n: src.tensor(n) * (6.0 if n.endswith("proj.weight") else 1.0) for n in src.names()}
        write_safetensors(str(tmp_path / "model.safetensors"), tensors)
        w = {n: t.numpy() for n, t in tensors.items()}
        engine = Engine.from_dir(str(tmp_path), EngineOptions(dtype="float32", kv_tokens=64, page_size=16, max_requests=3, record_after=1))
        assert engine.model.recordable and engine.model.native is None and engine.position_streams == 2 and not engine.cache.groups

        def plain_rows(ids, second, start, n):
            """The model on rows start .. start + n of a request: no token mixes with another, only the lengths count."""
            x = plain.embedding(w["model.embed_tokens.weight"], ids[start:start + n])
            length_after = start + n
            for b in (0, 1, 0):
                pre = f"model.layers.{b}."
                h = plain.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
                x = x + (h @ w[pre + "self_attn.proj.weight"].T) * np.float32(round(65536.0 / length_after) / 65536.0)
                x = x + np.asarray(second[start:start + n], dtype=np.float32)[:, None] * w[pre + "mlp.bias"][None, :] * np.float32(0.01)
            return plain.rms_norm(x, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T

        reqs = {r: (helpers.random_ids(V, 60, seed=s), helpers.random_ids(97, 60, seed=50 + s)) for r, s in (("p", 1), ("q", 2))}
        HistoryMeanMixer.plans.clear()
        for run in range(3):                     # the same shapes three times: plain, then recorded, then replayed
            at = {r: 0 for r in reqs}
            for counts in ((7, 3), (2, 1), (2, 1), (13, 5), (2, 1)):
                entries = []
                for (r, (ids, second)), n in zip(reqs.items(), counts):
                    entries.append(StepEntry(r, ids[at[r]:at[r] + n], list(range(n)), positions=[second[at[r]:at[r] + n]]))
                logits = engine.step(entries, record=True).float().cpu().numpy()
                k = 0
                for (r, (ids, second)), n in zip(reqs.items(), counts):
                    ref = plain_rows(ids, second, at[r], n)
                    assert np.abs(logits[k:k + n] - ref).max() <= 1e-4 * np.abs(ref).max(), (run, counts, r)
                    k += n
                    at[r] += n
            for r in reqs:
                engine.end(r)
        assert len(engine.step_recordings) == 3                                  # three shapes, each recorded once
        recorded = [p for p in HistoryMeanMixer.plans if p.recorded]
        assert len(recorded) == 6 and all(p.fills >= 2 for p in recorded)        # two mixers, three shapes: planned once each, filled every run
        with pytest.raises(Exception, match="positions must be 1 lists"):
            engine.step([StepEntry("z", [1, 2], [1], positions=[[5]])])
    finally:
        unregister_architecture(["PlannedToy", "planned_toy"])


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(64, 6, 2), (128, 8, 2), (128, 10, 2)])
def test_windowed_attention_in_bfloat16_with_pages_given_back_and_taken_again(head_dim, heads, kv_heads):
    """The tiled bfloat16 kernels under a window, through the cache manager: two requests take turns with portions
    that cross the window's edge and with decoded tokens, over a pool so small that the pages one gives back (its
    window has passed them; its block table then holds -1 there) are the pages the other takes.  The tiled prefill
    kernels start a stage below the window's first key, where those entries lie.  Every row against the plain
    mixer with the same window."""
    from llmx_b200 import ops_tc
    from llmx_b200.cache import CacheManager, KVSpec
    from llmx_b200.engine.batch import step_from_requests
    from llmx_b200.parts import Attention, Precision, RotaryEmbedding
    p = Precision.of("bfloat16")
    E, window, page = 64, 40, 16
    part = Attention(E, heads, kv_heads, head_dim, RotaryEmbedding(head_dim, 10000.0), qk_norm_eps=1e-6, window=window)
    g = torch.Generator().manual_seed(4)
    w = {n: (torch.randn(s.shape, generator=g) * (0.3 if s.kind == "matrix" else 0.1) + (0 if s.kind == "matrix" else 1)).to(p.act if s.kind == "matrix" else torch.float32)
         for n, s in part.tensor_specs().items()}
    part.load({n: t.to(DEV) for n, t in w.items()}, p)
    part.prepare(512, DEV)
    lengths = {"u": 230, "v": 190}
    hs = {r: torch.randn(n, E, generator=g).to(p.act) for r, n in lengths.items()}
    # a windowed request holds its window, the page it starts in and the portion being written: 2 x that, no more
    cache = CacheManager([KVSpec(kv_heads, head_dim, window)], page, 2 * (window + 2 * page + 48 + page), 2, kv_dtype=p.act, device=DEV)
    rcs = {r: cache.new_request(r) for r in lengths}
    got = {r: torch.zeros(n, E, device=DEV) for r, n in lengths.items()}
    at = {r: 0 for r in lengths}
    seen_released, given_back, taken_again = False, set(), False
    portions = {"u": [45, 1, 1, 37, 2, 48, 1, 3, 33, 1, 17, 41], "v": [1, 48, 2, 1, 29, 1, 40, 5, 1, 19, 43]}
    k = 0
    while any(at[r] < lengths[r] for r in lengths):
        who = [r for r in lengths if at[r] < lengths[r] and (k % 3 != 2 or r == "u")] or [r for r in lengths if at[r] < lengths[r]]
        counts = [min(portions[r][(k // 2) % len(portions[r])], lengths[r] - at[r]) for r in who]
        for r, n in zip(who, counts):
            rcs[r].prepare(n)
        held = {pg for r in who for pg in rcs[r].tables[0].pages if pg >= 0}
        taken_again = taken_again or bool(held & given_back)
        seen_released = seen_released or any(-1 in rcs[r].tables[0].pages for r in who)
        step = step_from_requests(cache, [rcs[r] for r in who], counts, DEV, parts=[part])
        h = torch.cat([hs[r][at[r]:at[r] + n] for r, n in zip(who, counts)]).to(DEV)
        res = torch.zeros(h.shape[0], E, device=DEV)
        part.forward(h, step, 0, res)
        a = 0
        for r, n in zip(who, counts):
            got[r][at[r]:at[r] + n] = res[a:a + n]
            a += n
            before = {pg for pg in rcs[r].tables[0].pages if pg >= 0}
            rcs[r].commit()
            given_back |= before - {pg for pg in rcs[r].tables[0].pages if pg >= 0}
            at[r] += n
        cache.check()
        k += 1
    torch.cuda.synchronize()
    ops_tc.check_errors()
    assert seen_released and taken_again, "the pool was not tight enough: no page was given back and taken again"
    cfg = dict(num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=1e-6)
    wf = {"p." + n: t.float().numpy() for n, t in w.items()}
    for r, n in lengths.items():
        cos, sin = plain.rope_tables(n, head_dim, 10000.0)
        ref = plain.attention_block(hs[r].float().numpy(), wf, "p.", cfg, cos, sin, act_round=plain.round_bf16, window=window)
        assert np.abs(got[r].cpu().numpy() - ref).max() <= 3e-2 * np.abs(ref).max(), r
