"""Configuration: every key read, defaults, and each refusal by message; the registry."""
import json

import pytest

from configs import TINY_A, TINY_B
from llmx_b200.config import ConfigError, Qwen3Config
from llmx_b200.registry import architecture_of, config_from_dir, register_architecture, unregister_architecture


def test_reads_every_size_from_config():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.intermediate_size) == (3, 96, 160)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 3, 32)
    assert c.q_width == 192 and c.kv_width == 96 and c.vocab_size == 384
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.rope_scaling.factor == 2.0 and c.rope_scaling.original_max_position_embeddings == 512
    assert abs(c.rope_scaling.attention_factor - 1.0693147) < 1e-6


def test_defaults():
    raw = dict(num_hidden_layers=1, hidden_size=64, intermediate_size=8, num_attention_heads=4, vocab_size=10)
    c = Qwen3Config.from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.max_position_embeddings == 4096 and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    assert c.rope_scaling is None and c.eos_ids == ()
    assert Qwen3Config.from_dict(dict(raw, eos_token_id=[3, 4])).eos_ids == (3, 4)


def test_round_trip_through_to_dict():
    for raw in (TINY_A, TINY_B):
        c = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict()))) == c


@pytest.mark.parametrize("change,message", [
    (dict(bogus_key=1), "unknown config.json key"),
    (dict(num_hidden_layers=0), "num_hidden_layers must be an integer >= 1"),
    (dict(hidden_size=64.0), "hidden_size must be an integer"),
    (dict(num_attention_heads=True), "num_attention_heads must be an integer"),
    (dict(num_key_value_heads=3), "divisible by KV head count"),
    (dict(head_dim=15), "head_dim must be even"),
    (dict(attention_bias=True), "attention_bias must be one of"),
    (dict(hidden_act="gelu"), "hidden_act must be one of"),
    (dict(use_sliding_window=True), "use_sliding_window must be one of"),
    (dict(layer_types=["full_attention", "sliding_attention"]), "every entry of layer_types"),
    (dict(torch_dtype="int8"), "torch_dtype must be one of"),
    (dict(rope_theta="big"), "rope_theta must be a finite number"),
    (dict(rope_scaling={"factor": 2.0}), "gives no rope_type"),
    (dict(rope_scaling={"rope_type": "linear", "factor": 2.0}), "is not supported"),
    (dict(rope_scaling={"rope_type": "yarn"}), "gives no factor"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 1.0}), "factor must be above 1"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2.0, "mscale": 1.0}), "mscale is not supported"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2.0, "beta_fast": 1.0, "beta_slow": 2.0}), "beta_fast must be above"),
    (dict(architectures=["LlamaForCausalLM"]), "architectures"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings must be true or false"),
])
def test_refusals(change, message):
    raw = dict(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    assert message in str(e.value)


def test_missing_keys_are_listed():
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(hidden_size=64))
    assert "num_hidden_layers" in str(e.value) and "vocab_size" in str(e.value)


def test_head_dim_must_divide_when_absent():
    raw = {k: v for k, v in TINY_A.items() if k != "head_dim"}
    raw["hidden_size"] = 66
    with pytest.raises(ConfigError):
        Qwen3Config.from_dict(raw)


def test_registry_by_class_name_and_model_type(tmp_path):
    assert architecture_of({"architectures": ["Qwen3ForCausalLM"]}).config_cls is Qwen3Config
    assert architecture_of({"model_type": "qwen3"}).config_cls is Qwen3Config
    with pytest.raises(ConfigError) as e:
        architecture_of({"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2"})
    assert "GPT2LMHeadModel" in str(e.value) and "qwen3" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    entry, cfg = config_from_dir(str(tmp_path))
    assert entry.name == "Qwen3ForCausalLM" and cfg.hidden_size == 64
    model = entry.build(cfg)
    assert len(model.blocks) == 2 and model.vocab_size == 256
    with pytest.raises(ConfigError):
        config_from_dir(str(tmp_path / "nothing"))


def test_registering_another_architecture():
    calls = []
    register_architecture(["ToyForCausalLM", "toy"], Qwen3Config, lambda c: calls.append(c) or "model")
    try:
        assert architecture_of({"model_type": "toy"}).build("cfg") == "model" and calls == ["cfg"]
        with pytest.raises(ValueError):
            register_architecture(["toy"], Qwen3Config, lambda c: None)
    finally:
        unregister_architecture(["ToyForCausalLM", "toy"])


def test_matrix_product_plan_fills_the_sms():
    """The host-side choice of schedule, token tile and k ranges (a pure function of the shape)."""
    from llmx_b200 import ops_tc
    sms = 148
    # few tokens: stream-K; the logits head has tiles enough and keeps whole tiles, unsplit
    assert ops_tc._plan(8, 4096, 4096, True, sms) == (1, 0, 1)
    assert ops_tc._plan(8, 151936, 4096, False, sms) == (0, 0, 1)
    # a few hundred tokens on a [4096, 4096] weight: 32 to 64 tiles would idle most SMs, so K is cut; whole tiles run on
    # single blocks (schedule 0: 128 weight rows a tile) or on pairs of SMs (schedule 2: 256 weight rows a pair)
    for m in (96, 128, 256, 512):
        schedule, tile, splits = ops_tc._plan(m, 4096, 4096, True, sms)
        assert schedule in (0, 2) and tile in (128, 256)
        units = -(-4096 // (256 if schedule == 2 else 128)) * -(-m // tile) * splits
        assert units >= (48 if schedule == 2 else 96)          # of 74 pairs, of 148 blocks
        assert splits >= 2 or units >= (64 if schedule == 2 else 128)
    from llmx_b200 import runtime
    before = runtime.pair_products(False)
    try:
        for m in (96, 128, 256, 512):
            schedule, tile, splits = ops_tc._plan(m, 4096, 4096, True, sms)
            assert schedule == 0 and tile in (128, 256) and splits >= 2
            assert -(-4096 // 128) * -(-m // tile) * splits >= 96
    finally:
        runtime.pair_products(before)
    # 33 to 64 tokens: whole tiles of 64 tokens with K in equal ranges where those still fill three quarters of the 296
    # blocks that run at once (fewer pieces to add up than stream-K makes); else stream-K, as up to 32 tokens
    assert ops_tc._plan(64, 4096, 4096, True, sms) == (0, 64, 8)
    assert ops_tc._plan(40, 6144, 4096, False, sms) == (0, 64, 6)
    assert ops_tc._plan(64, 24576, 4096, False, sms) == (1, 0, 1)          # 192 tiles: one range each would leave a third of the blocks idle
    assert ops_tc._plan(32, 4096, 4096, True, sms) == (1, 0, 1)
    # many tokens on pairs of SMs: where the tiles leave a partial last round (128 pair tiles on 74 pairs), only that
    # round's tiles are cut (splits 0), and only for a product that adds to its output or is cleared first
    assert ops_tc._plan(2048, 4096, 12288, True, sms) == (2, 256, 0)
    assert ops_tc._plan(8192, 4096, 12288, True, sms) == (2, 256, 1)        # 512 tiles: 6.9 rounds, nothing to cut
    # many tokens: whole tiles fill the SMs by themselves
    assert ops_tc._plan(4096, 6144, 4096, False, sms)[2] == 1
    # k ranges never outnumber the k blocks
    assert ops_tc._plan(128, 4096, 64, True, sms)[2] == 1


def test_attention_shapes_fill_the_sms():
    """The host-side choices for attention (pure functions of the step's shape): row tiles an item and key ranges
    for prompt portions, key ranges for decoding rows, weight rows a tile for the q/k/v product."""
    from llmx_b200 import ops_attn, ops_tc
    # a whole prompt makes items enough: pairs of row tiles, all keys
    assert ops_attn.prefill_shape(1, 8, 4, 2048, 2048, 0) == (2, 1)
    # a short portion: fewer pairs than half the SMs, so single tiles; few key stages, so no ranges
    assert ops_attn.prefill_shape(1, 8, 4, 256, 256, 0) == (1, 1)
    # a portion after a long history: the keys are cut into ranges, more of them the fewer the items
    tiles, ranges = ops_attn.prefill_shape(1, 8, 4, 512, 4608, 0)
    assert ranges >= 2
    assert ops_attn.prefill_shape(1, 8, 4, 256, 8448, 0)[1] > ranges
    # a window bounds the keys an item walks, whatever the history
    assert ops_attn.prefill_shape(1, 8, 4, 512, 40000, 512)[1] == 1
    # the partial results stay within their bound
    for rows, ctx in ((512, 4608), (2048, 40000), (8192, 40000)):
        t, r = ops_attn.prefill_shape(4, 8, 4, rows, ctx, 0)
        assert r == 1 or rows * 32 * 4 * r * ops_attn.PREFILL_PART <= ops_attn.PREFILL_MAX_PARTIAL
    # decoding rows: a range per 128 keys at first, then as many as fit as clusters (eight at most below 4,096 keys,
    # sixteen above); never more blocks than a wave
    assert ops_attn.decode_schedule(8, 8, 100)[0] == 1 and ops_attn.decode_schedule(1, 8, 512)[0] == 4
    assert ops_attn.decode_schedule(1, 8, 2048)[0] == 8 and ops_attn.decode_schedule(1, 8, 8192)[0] == 16
    assert ops_attn.decode_schedule(2, 8, 8192)[0] == 8 and ops_attn.decode_schedule(2, 8, 32768)[0] == 12
    assert ops_attn.decode_schedule(8, 8, 8192)[0] == 4 and ops_attn.decode_schedule(64, 8, 8192)[0] == 1
    for n, ctx in ((1, 8192), (8, 8192), (64, 8192), (4, 32768)):
        splits, chunk = ops_attn.decode_schedule(n, 8, ctx)
        assert splits * chunk >= ctx and chunk % 64 == 0 and (splits == 1 or n * 8 * splits <= ops_attn.WAVE_BLOCKS)
    # the q/k/v product finishes its heads itself from 256 rows on
    ops_tc._sm_count = ops_tc._sm_count or 148
    assert ops_tc.heads_tile(255, 32, 8) == 0 and ops_tc.heads_tile(256, 32, 8) in (128, 256)
    assert ops_tc.heads_tile(2048, 32, 8) == 256


def test_yarn_forced_over_the_files_rope():
    """--yarn F [--yarn-original-ctx N]: the length it scales is N, else the files' declared original, else their
    context; the context becomes F times that; the files' betas stay when they declare YaRN themselves."""
    plain = Qwen3Config.from_dict(TINY_A)                       # no rope_scaling, context 512
    c = plain.with_yarn(4.0)
    assert c.rope_scaling.factor == 4.0 and c.rope_scaling.original_max_position_embeddings == 512
    assert c.max_position_embeddings == 2048 and (c.rope_scaling.beta_fast, c.rope_scaling.beta_slow) == (32.0, 1.0)
    c = plain.with_yarn(2.5, 100)
    assert c.rope_scaling.original_max_position_embeddings == 100 and c.max_position_embeddings == 250
    declared = Qwen3Config.from_dict(dict(TINY_B, rope_scaling=dict(rope_type="yarn", factor=2.0, beta_fast=16.0,
                                                                    original_max_position_embeddings=512)))
    c = declared.with_yarn(3.0)
    assert c.rope_scaling.original_max_position_embeddings == 512 and c.max_position_embeddings == 1536
    assert c.rope_scaling.beta_fast == 16.0
    for bad in (1.0, 0.5, float("inf"), float("nan")):
        with pytest.raises(ConfigError):
            plain.with_yarn(bad)
    with pytest.raises(ConfigError) as e:
        plain.with_yarn(2.0, 513)
    assert "past the model's context of 512" in str(e.value)
    # the command line's two flags
    from llmx_b200.cli.main import UsageError, _yarn
    assert _yarn({}) == (None, None) and _yarn({"--yarn": "4", "--yarn-original-ctx": "128"}) == (4.0, 128)
    for given in ({"--yarn": "1"}, {"--yarn": "0.5"}, {"--yarn-original-ctx": "128"}, {"--yarn": "2", "--yarn-original-ctx": "0"}):
        with pytest.raises(UsageError):
            _yarn(given)


def test_a_rebuilt_library_removes_its_own_older_builds_only(tmp_path):
    """Build files are `llmx_<library>_<16 hex digits>.so`; `gemm_tc_pair` and `attention_prefill_tc` are libraries of
    their own, not older builds of `gemm_tc` and `attention_prefill`."""
    from llmx_b200.csrc import build
    names = ["llmx_gemm_tc_0123456789abcdef.so", "llmx_gemm_tc_fedcba9876543210.so", "llmx_gemm_tc_pair_0123456789abcdef.so",
             "llmx_attention_prefill_tc_0123456789abcdef.so", "llmx_gemm_tc_0123456789abcdef.so.123.tmp", "notes.txt"]
    for n in names:
        (tmp_path / n).write_bytes(b"")
    build._remove_older_builds("gemm_tc", str(tmp_path / "llmx_gemm_tc_fedcba9876543210.so"))
    assert sorted(p.name for p in tmp_path.iterdir()) == sorted(n for n in names if n != "llmx_gemm_tc_0123456789abcdef.so")
    build._remove_older_builds("attention_prefill", str(tmp_path / "llmx_attention_prefill_0000000000000000.so"))
    assert (tmp_path / "llmx_attention_prefill_tc_0123456789abcdef.so").exists()


def test_bench_refuses_more_than_one_gpu_in_one_line():
    """`bench.py --gpus N` for N > 1: one line that says so, exit code 2, before anything of CUDA is touched."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    done = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert done.returncode == 2
    assert len(done.stdout.strip().splitlines()) == 1 and "one GPU" in done.stdout
