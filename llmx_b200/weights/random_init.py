"""The random-weights mode: a model's tensors from a configuration and a seed.

Matrices and embeddings are N(0, 0.02); norm weights are 1 + N(0, 0.01), so a
norm's weight is never mistaken for the identity.  The generator is counter-based:
element i of a tensor is a function of (seed, tensor name, i) alone -- a 64-bit mix of the three picks one of
2^20 quantiles of the standard normal from a table made once on the host -- so a tensor's values do not depend on
which other tensors exist, on the order they are made in, or on the device that makes them: "seed 0" names
one model, whether its weights are made on the GPU for a benchmark or on the CPU for a model folder.  The reference's
own synthetic model (src/model/arch/qwen3.hpp:332-397) is a uniform(-1, 1)
mt19937 fill used only for timing; this one is made to be written out and read
back as an ordinary model folder.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .safetensors import write_safetensors
from .spec import TensorSpec


def _stream_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


_QUANTILE_BITS = 20
_tables: Dict[str, torch.Tensor] = {}


def _quantiles(device: torch.device) -> torch.Tensor:
    """The standard normal's quantiles at (k + 0.5) / 2^20, float32: computed in float64 on the host, the same
    values then serve every device."""
    key = str(device)
    if key not in _tables:
        if "cpu" not in _tables:
            n = 1 << _QUANTILE_BITS
            u = (torch.arange(n, dtype=torch.float64) + 0.5) / n
            _tables["cpu"] = torch.special.ndtri(u).to(torch.float32)
        _tables[key] = _tables["cpu"].to(device)
    return _tables[key]


def _mix64(x: torch.Tensor) -> torch.Tensor:
    """splitmix64's finaliser on int64 values (arithmetic wraps; shifts are made logical by masking)."""
    def shr(v, k):
        return (v >> k) & ((1 << (64 - k)) - 1)
    x = (x ^ shr(x, 30)) * -4658895280553007687          # 0xBF58476D1CE4E5B9 as a signed 64-bit value
    x = (x ^ shr(x, 27)) * -7723592293110705685          # 0x94D049BB133111EB
    return x ^ shr(x, 31)


def standard_normal(stream: int, count: int, device: torch.device, chunk: int = 1 << 26) -> torch.Tensor:
    """`count` float32 values of the stream `stream`: value i = quantile[top 20 bits of mix64(stream + golden * i)]."""
    table = _quantiles(device)
    out = torch.empty(count, dtype=torch.float32, device=device)
    base = torch.tensor(stream, dtype=torch.int64, device=device)
    for at in range(0, count, chunk):
        n = min(chunk, count - at)
        i = torch.arange(at, at + n, dtype=torch.int64, device=device)
        h = _mix64(base + i * -7046029254386353131)      # 0x9E3779B97F4A7C15, the counter's stride
        out[at:at + n] = table[(h >> (64 - _QUANTILE_BITS)) & ((1 << _QUANTILE_BITS) - 1)]
    return out


class RandomSource:
    """A tensor source that makes each tensor on demand from (seed, name)."""

    def __init__(self, specs: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                 device: str = "cpu", skip_optional: bool = False):
        self.specs = {n: s for n, s in specs.items() if not (skip_optional and s.optional)}
        self.seed = int(seed)
        self._dtype = dtype
        self.device = torch.device(device)

    def names(self) -> List[str]:
        return list(self.specs)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.specs[name].shape)

    def dtype(self, name: str) -> torch.dtype:
        s = self.specs[name]
        if s.kind == "int_table":
            return torch.int32
        return torch.float32 if s.kind == "vector" else self._dtype

    def tensor(self, name: str) -> torch.Tensor:
        s = self.specs[name]
        stream = _stream_seed(self.seed, name)
        count = 1
        for d in s.shape:
            count *= int(d)
        if s.kind == "int_table":
            i = torch.arange(count, dtype=torch.int64, device=self.device)
            h = _mix64(torch.tensor(stream, dtype=torch.int64, device=self.device) + i * -7046029254386353131)
            return ((h >> 49) & 0x7FFF).to(torch.int32).reshape(tuple(s.shape))
        # One multiplication and one addition, each rounded once: the same bits on every device.
        t = standard_normal(stream, count, self.device) * s.std
        if s.init == "one_plus_normal":
            t = t + 1.0
        return t.reshape(tuple(s.shape)).to(self.dtype(name))


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write config.json and model.safetensors for `config` with random weights.

    The model class is chosen from the configuration by the registry, as
    everywhere.  Returns the folder.
    """
    from ..registry import architecture_of

    raw = config.to_dict()
    entry = architecture_of(raw)
    model = entry.build(config)
    specs = model.tensor_specs()
    src = RandomSource(specs, seed, dtype=dtype, device="cpu", skip_optional=True)
    os.makedirs(model_dir, exist_ok=True)
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1, sort_keys=True)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      {n: src.tensor(n) for n in src.names()},
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
