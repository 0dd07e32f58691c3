"""Tiny configurations of the architecture for the tests.

A and B differ in every size and option: layers, widths, head counts and group
ratio, head width, vocabulary, rope base, eps, tying, context, page size, and B
has YaRN rope scaling (a frequency blend and an attention factor).  They are BASELINE.json's
tiny A and tiny B with a longer context (and B's YaRN); BASELINE_A and BASELINE_B below are those to the letter.  C has widths
the tensor-core path cannot take (an input width that is no multiple of 8), a
head width of 48 and an odd vocabulary.
"""
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=512, eos_token_id=255)

TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, intermediate_size=160, num_attention_heads=6, num_key_value_heads=3,
    head_dim=32, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
    max_position_embeddings=1024,
    rope_scaling=dict(rope_type="yarn", factor=2.0, original_max_position_embeddings=512, beta_fast=32.0, beta_slow=1.0))

TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=100, intermediate_size=172, num_attention_heads=3, num_key_value_heads=1,
    head_dim=48, vocab_size=257, rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=512)

# D has the head width and page size the tiled bfloat16 attention kernels take, so the serving kernels
# (tensor-core products, split-KV decode, tiled prefill) run under every cutting too.
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=128, intermediate_size=200, num_attention_heads=6, num_key_value_heads=2,
    head_dim=64, vocab_size=320, rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=2048)

# E has a head ratio that divides neither 16 nor 128 (five query heads a kv head, as Qwen3-14B's 40 over 8) at the
# head width of the tensor-core attention, so a decoding request fills a 16-row tile with three rows and a prompt
# portion's row tile holds 25 tokens and three rows of padding.
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=192, intermediate_size=264, num_attention_heads=10, num_key_value_heads=2,
    head_dim=128, vocab_size=300, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=2048)

CONFIGS = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16), "D": (TINY_D, 3, 16),
           "E": (TINY_E, 4, 16)}   # config, seed, page size

# BASELINE.json's tiny A and tiny B to the letter.  A and B above are these with a longer context (512 and 1,024
# instead of 128 and 256 positions, so that prompts of 133 tokens fit the cuttings) and, for B, a YaRN rope scaling
# BASELINE's B does not declare (so that the scaled rope is under every cutting too): more is tested, not less.
# These two run BASELINE's own workloads (tests/test_generate_gpu.py).
BASELINE_A = dict(TINY_A, max_position_embeddings=128)
BASELINE_B = {k: v for k, v in dict(TINY_B, max_position_embeddings=256).items() if k != "rope_scaling"}


# What the bfloat16 path may differ from the plain implementation that rounds the same things (inputs of products,
# queries, the cache), as a fraction of the logit scale: twice the error measured for each configuration when the
# budget was frozen (A 5.3e-4, B 4.4e-3, C 1.8e-3, D 2.6e-3, E 4.0e-3, two layers of Qwen3-8B's width 7.6e-3; the same
# under every cutting, since it is the kernels' own rounding -- bfloat16 softmax weights, the order of sums -- that is
# measured).  The reference budgets its reduced-precision paths the same way (docs/PRECISION.md:99-118).  A budget is
# not widened to make a test pass.  "sharp:X": the same model with q/k norm weights doubled (scores spread four times
# as wide, so a key read from the wrong place shows).
BF16_BUDGET = {"A": 1.1e-3, "B": 9e-3, "C": 3.6e-3, "D": 5.2e-3, "E": 8.2e-3, "wide": 1.6e-2,
               "sharp:B": 1.5e-2, "sharp:D": 1.5e-2, "sharp:E": 1.7e-2}
BF16_UNCALIBRATED = 1e-2           # configurations made inside single tests
