"""The reference arm of bench.py: the unmodified mxxm-t/llmx, built with its own CMake, timed by its own `llmx bench`.

    python bench.py --impl reference [--steps K] [--size 8b] [--batch 8] [--context 8192]

What runs is the reference's stock measurement (src/cli/main.cpp:1192-1287, `cmd_bench_model`) on its CUDA
backend (`--device cuda:0`; the kernels are its own, from PTX for compute_80 that the driver compiles for the
device, docs/CUDA.md) over a model folder of the same configuration as bench.py's own arm: random bfloat16
weights N(0, 0.02) in `model.safetensors`, the same config.json keys, and the smallest tokenizer files its
loader accepts (src/tokenizer/hf_tokenizer.hpp:114-146; the bench feeds fixed ids and never tokenizes).
Nothing of llmx_b200 is imported or loaded here.

Two runs of the binary give the two numbers:
  prefill   `llmx bench --model DIR --p 2048 --n 4 --r R`          -> "bench: pp2048 ... tok/s"
  decode    `llmx bench --model DIR --p CONTEXT --n K --r R --seqs B` -> "bench: xB tgK ... tok/s"
            (with several sequences its decode follows each sequence's prompt, so the prompt length is the
            context; `--depth` takes one sequence only, src/cli/main.cpp:2214)
Its clock is the host's around whole passes with the logits read each step (its `e2e` and its `value` are the
same number: it has no device-only timer).

The binary is expected at baseline/_ref/build/llmx, built by
    cmake -S <reference> -B baseline/_ref/build -DLLMX_HAS_BACKEND_CUDA=ON -DBUILD_TESTING=OFF -DCMAKE_BUILD_TYPE=Release
    make -C baseline/_ref/build llmx
When it is missing and the reference's source tree is at hand it is built first; when neither is there, or a step
fails, one line `{"impl": "reference", "unavailable": "<why>"}` is printed and the exit code is 0.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import shutil
import struct
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "baseline", "_ref", "build")
BINARY = os.path.join(BUILD, "llmx")
SOURCE = os.environ.get("LLMX_REFERENCE_SOURCE", "/root/reference")

# The Split pattern the reference's tokenizer reader insists on (src/tokenizer/hf_tokenizer.hpp:22-23).
QWEN2_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")


class Unavailable(Exception):
    pass


def _say(text: str) -> None:
    print(f"[reference arm] {text}", file=sys.stderr, flush=True)


def build_binary() -> str:
    if os.path.isfile(BINARY) and os.access(BINARY, os.X_OK):
        return BINARY
    if not os.path.isfile(os.path.join(SOURCE, "CMakeLists.txt")):
        raise Unavailable(f"no reference binary at baseline/_ref/build/llmx and no source tree at {SOURCE} to build it from")
    os.makedirs(BUILD, exist_ok=True)
    _say("building the reference (cmake, CUDA backend): several minutes")
    for cmd in (["cmake", "-S", SOURCE, "-B", BUILD, "-DLLMX_HAS_BACKEND_CUDA=ON", "-DBUILD_TESTING=OFF",
                 "-DCMAKE_BUILD_TYPE=Release"],
                ["make", "-C", BUILD, f"-j{os.cpu_count() or 4}", "llmx"]):
        try:
            done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=3000)
        except (OSError, subprocess.TimeoutExpired) as e:
            raise Unavailable(f"building the reference failed: {cmd[0]}: {e}") from None
        if done.returncode != 0:
            raise Unavailable(f"building the reference failed: {cmd[0]} exit {done.returncode}: "
                              + " | ".join(done.stdout.strip().splitlines()[-3:]))
    return BINARY


# ---------------------------------------------------------------------------------------------------------------
def _tensor_list(cfg: dict):
    """(name, shape) of every tensor of a dense Qwen3 checkpoint, in file order."""
    E, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    D = cfg["head_dim"]
    Q, KV = cfg["num_attention_heads"] * D, cfg["num_key_value_heads"] * D
    out = [("model.embed_tokens.weight", (V, E))]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (E,)), (p + "self_attn.q_proj.weight", (Q, E)),
                (p + "self_attn.k_proj.weight", (KV, E)), (p + "self_attn.v_proj.weight", (KV, E)),
                (p + "self_attn.q_norm.weight", (D,)), (p + "self_attn.k_norm.weight", (D,)),
                (p + "self_attn.o_proj.weight", (E, Q)), (p + "post_attention_layernorm.weight", (E,)),
                (p + "mlp.gate_proj.weight", (F, E)), (p + "mlp.up_proj.weight", (F, E)),
                (p + "mlp.down_proj.weight", (E, F))]
    out.append(("model.norm.weight", (E,)))
    if not cfg.get("tie_word_embeddings", False):
        out.append(("lm_head.weight", (V, E)))
    return out


def write_model_folder(cfg: dict, folder: str) -> None:
    """config.json, model.safetensors (bfloat16: matrices N(0, 0.02), norm weights 1 + N(0, 0.01), seed 0) and the
    tokenizer files, written tensor by tensor (the 8B file is 16 GB)."""
    import torch
    os.makedirs(folder, exist_ok=True)
    tensors = _tensor_list(cfg)
    header, at = {}, 0
    for name, shape in tensors:
        n = 2
        for s in shape:
            n *= s
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [at, at + n]}
        at += n
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=device)
    gen.manual_seed(0)
    started = time.time()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for k, (name, shape) in enumerate(tensors):
            if len(shape) == 1:
                t = 1.0 + 0.01 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
            else:
                t = 0.02 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
            raw = t.to(torch.bfloat16).view(torch.int16).cpu().numpy()
            f.write(memoryview(raw).cast("B"))
            if time.time() - started > 20:
                _say(f"writing weights: {k + 1} of {len(tensors)} tensors")
                started = time.time()
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    # The smallest byte-level BPE the loader takes: 256 single-byte tokens, no merges, one added end token.
    def byte_token(b: int) -> str:
        # the GPT-2 byte-to-character table: printable bytes stand for themselves, the rest are moved above U+0100
        printable = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
        if b in printable:
            return chr(b)
        others = [x for x in range(256) if x not in printable]
        return chr(256 + others.index(b))
    vocab = {byte_token(b): b for b in range(256)}
    end = {"id": 256, "content": "<|endoftext|>", "single_word": False, "lstrip": False, "rstrip": False,
           "normalized": False, "special": True}
    byte_level = {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": False, "use_regex": False}
    tokenizer = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [end],
                 "normalizer": {"type": "NFC"},
                 "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
                     {"type": "Split", "pattern": {"Regex": QWEN2_SPLIT}, "behavior": "Isolated", "invert": False},
                     byte_level]},
                 "post_processor": None, "decoder": byte_level,
                 "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": "",
                           "end_of_word_suffix": "", "fuse_unk": False, "byte_fallback": False, "ignore_merges": False,
                           "vocab": vocab, "merges": []}}
    with open(os.path.join(folder, "tokenizer.json"), "w") as f:
        json.dump(tokenizer, f)
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"add_bos_token": False, "add_eos_token": False, "eos_token": "<|endoftext|>",
                   "pad_token": "<|endoftext|>", "clean_up_tokenization_spaces": False, "errors": "replace",
                   "split_special_tokens": False, "tokenizer_class": "Qwen2Tokenizer"}, f)
    with open(os.path.join(folder, "complete"), "w") as f:
        f.write("ok\n")


def model_folder(cfg: dict) -> str:
    """A folder holding the model, written once per configuration under the temporary directory."""
    key = hashlib.sha1(json.dumps(cfg, sort_keys=True).encode()).hexdigest()[:12]
    params = sum(_prod(s) for _, s in _tensor_list(cfg))
    need = 2 * params + (64 << 20)
    for base in (tempfile.gettempdir(), "/dev/shm"):
        folder = os.path.join(base, f"llmx_reference_model_{key}")
        if os.path.exists(os.path.join(folder, "complete")):
            return folder
        try:
            free = shutil.disk_usage(base).free
        except OSError:
            continue
        if free > need + (2 << 30):
            if os.path.isdir(folder):
                shutil.rmtree(folder)
            _say(f"writing a {2 * params / 1e9:.1f} GB model folder to {folder}")
            write_model_folder(cfg, folder)
            return folder
    raise Unavailable(f"no room for a {need / 1e9:.0f} GB model folder under {tempfile.gettempdir()} or /dev/shm")


def _prod(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


# ---------------------------------------------------------------------------------------------------------------
RATE = re.compile(r"bench:\s+(x\d+ )?(pp|tg)(\d+)(?: @ d\d+)?\s+([0-9.]+) \+- ([0-9.]+) tok/s\s+\((\d+) runs\)")


def run_bench(binary: str, folder: str, flags, timeout: float):
    cmd = [binary, "bench", "--model", folder, "--device", "cuda:0"] + [str(x) for x in flags]
    _say(" ".join(cmd))
    t0 = time.time()
    try:
        done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        raise Unavailable(f"the reference's bench did not finish within {timeout:.0f} s: {' '.join(cmd[1:])}") from None
    except OSError as e:
        raise Unavailable(f"the reference binary does not start: {e}") from None
    if done.returncode != 0:
        tail = " | ".join((done.stderr.strip() or done.stdout.strip()).splitlines()[-3:])
        raise Unavailable(f"the reference's bench exited {done.returncode}: {tail}")
    rates = {}
    for line in done.stdout.splitlines():
        m = RATE.search(line)
        if m:
            rates[m.group(2)] = {"value": float(m.group(4)), "sd": float(m.group(5)), "runs": int(m.group(6)),
                                 "tokens": int(m.group(3))}
    notes = [l.strip() for l in (done.stdout + "\n" + done.stderr).splitlines() if l.startswith(("dtype:", "device", "plan"))]
    return rates, notes, time.time() - t0, done.stdout


def main(args, cfg: dict, size_name: str) -> int:
    """`args`: bench.py's parsed arguments; `cfg`: the config.json of the model both arms run."""
    try:
        binary = build_binary()
        folder = model_folder(cfg)
        repeats = 3
        pre, notes, pre_s, _ = run_bench(binary, folder, ["--p", args.prefill_tokens, "--n", 4, "--r", repeats], 1500)
        if "pp" not in pre:
            raise Unavailable("the reference's bench printed no pp line")
        flags = ["--p", args.context, "--n", args.steps, "--r", 1]
        if args.batch > 1:
            flags += ["--seqs", args.batch]
        dec, notes2, dec_s, out = run_bench(binary, folder, flags, 3000)
        if "tg" not in dec:
            raise Unavailable("the reference's bench printed no tg line: " + " | ".join(out.strip().splitlines()[-2:]))
    except Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    value = dec["tg"]["value"]
    ms = args.batch * 1e3 / value
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} (Qwen3-{size_name.upper()} sizes, bf16, random weights)",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": 1,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights; activations as the reference's --dtype auto resolves (see notes)", "data": "synthetic",
        "impl": "reference", "same_config": True,
        "config": {"model": f"Qwen3-{size_name.upper()} sizes, random weights", "layers": cfg["num_hidden_layers"],
                   "model_layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": args.context, "prefill_tokens": args.prefill_tokens,
                   "parallelism": "single GPU", "command": "llmx bench --model DIR --device cuda:0",
                   "timer": "host clock around whole passes, logits read every step",
                   "history": "each sequence's own prompt of seq_len tokens"},
        "e2e": {"value": round(value, 2), "unit": "tok/s", "ms_per_step": round(ms, 4),
                "note": "the reference's bench times on the host through its public Model::forward; one number"},
        "prefill": {"value": pre["pp"]["value"], "sd": pre["pp"]["sd"], "runs": pre["pp"]["runs"],
                    "tokens": pre["pp"]["tokens"], "ms": round(pre["pp"]["tokens"] * 1e3 / pre["pp"]["value"], 3)},
        "decode_sd": dec["tg"]["sd"], "wall_s": {"prefill_run": round(pre_s, 1), "decode_run": round(dec_s, 1)},
        "notes": (notes + notes2)[:6],
    }
    print(json.dumps(line))
    return 0
