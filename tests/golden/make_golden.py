#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of mxxm-t/llmx's own CPU float32 code on tiny random models.

Run by hand where a checkout of mxxm-t/llmx is at hand:
    REFERENCE=/path/to/llmx python tests/golden/make_golden.py
It writes each tiny model's weights with this repository's random-weights mode, compiles
tests/golden/reference_driver.cpp against the reference's headers (CPU only), runs it, and stores
the token ids and the reference's logits (whole prompt and token by token).  tests/test_plain.py
compares the plain implementation with these files; nothing at test time needs the reference.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
REFERENCE = os.environ.get("REFERENCE")
if not REFERENCE:
    sys.exit("set REFERENCE to a checkout of mxxm-t/llmx")

from configs import TINY_A, TINY_B  # noqa: E402
from llmx_b200.config import Qwen3Config  # noqa: E402
from llmx_b200.weights import RandomSource  # noqa: E402
from llmx_b200.registry import architecture_of  # noqa: E402

NAMES = {"input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "self_attn.q_norm": "attn_q_norm",
         "self_attn.k_norm": "attn_k_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
         "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate",
         "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}


def internal_name(hf: str) -> str:
    if hf == "model.embed_tokens.weight":
        return "token_embd.weight"
    if hf == "model.norm.weight":
        return "output_norm.weight"
    if hf == "lm_head.weight":
        return "output.weight"
    parts = hf.split(".")
    layer, rest = parts[2], ".".join(parts[3:-1])
    return f"blk.{layer}.{NAMES[rest]}.weight"


def main():
    work = tempfile.mkdtemp()
    exe = os.path.join(work, "reference_driver")
    cmd = ["g++", "-std=c++17", "-O1", "-ffp-contract=off", "-mavx2", "-mfma", "-mf16c", "-pthread",
           f"-I{REFERENCE}/src", f"-I{REFERENCE}/tests", os.path.join(HERE, "reference_driver.cpp"), "-o", exe]
    print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    for tag, raw, seed in (("tiny_a", TINY_A, 0), ("tiny_b", TINY_B, 1)):
        cfg = Qwen3Config.from_dict(raw)
        model = architecture_of(cfg.to_dict()).build(cfg)
        src = RandomSource(model.tensor_specs(), seed, dtype=torch.float32, skip_optional=True)
        meta = [("block_count", "u32", cfg.num_hidden_layers), ("embedding_length", "u32", cfg.hidden_size),
                ("feed_forward_length", "u32", cfg.intermediate_size), ("attention.head_count", "u32", cfg.num_attention_heads),
                ("attention.head_count_kv", "u32", cfg.num_key_value_heads), ("attention.key_length", "u32", cfg.head_dim),
                ("context_length", "u32", cfg.max_position_embeddings), ("rope.freq_base", "f32", repr(cfg.rope_theta)),
                ("attention.layer_norm_rms_epsilon", "f32", repr(cfg.rms_norm_eps))]
        if cfg.rope_scaling is not None:
            y = cfg.rope_scaling
            meta += [("rope.scaling.type", "str", "yarn"), ("rope.scaling.factor", "f32", repr(y.factor)),
                     ("rope.scaling.original_context_length", "u32", y.original_max_position_embeddings),
                     ("rope.scaling.yarn_beta_fast", "f32", repr(y.beta_fast)),
                     ("rope.scaling.yarn_beta_slow", "f32", repr(y.beta_slow))]
        with open(os.path.join(work, "meta.txt"), "w") as f:
            for k, t, v in meta:
                f.write(f"{k} {t} {v}\n")
        at, chunks, lines = 0, [], []
        for name in src.names():
            t = src.tensor(name).to(torch.float32).contiguous().numpy()
            ne = list(reversed(t.shape))          # fastest dimension first
            lines.append(f"{internal_name(name)} {len(ne)} {' '.join(map(str, ne))} {at}")
            chunks.append(t.reshape(-1))
            at += t.size
        with open(os.path.join(work, "manifest.txt"), "w") as f:
            f.write("\n".join(lines) + "\n")
        np.concatenate(chunks).astype("<f4").tofile(os.path.join(work, "weights.bin"))
        ids = np.random.default_rng(seed + 10).integers(0, cfg.vocab_size, size=24)
        with open(os.path.join(work, "ids.txt"), "w") as f:
            f.write(" ".join(map(str, ids.tolist())))
        subprocess.run([exe] + [os.path.join(work, n) for n in ("meta.txt", "manifest.txt", "weights.bin", "ids.txt", "out.bin")],
                       check=True)
        out = np.fromfile(os.path.join(work, "out.bin"), dtype="<f4").reshape(2, len(ids), cfg.vocab_size)
        np.savez_compressed(os.path.join(HERE, f"{tag}.npz"), ids=ids.astype(np.int32), seed=np.int32(seed),
                            whole=out[0], steps=out[1])
        print(tag, "whole-vs-steps maxabs", float(np.abs(out[0] - out[1]).max()))


if __name__ == "__main__":
    main()
