"""The random-weights mode: a model's tensors from a configuration and a seed.

Matrices and embeddings are N(0, 0.02); norm weights are 1 + N(0, 0.01), so a
norm's weight is never mistaken for the identity.  Each tensor has its own
stream keyed by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist or on the order they are made in.  The reference's
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
        g = torch.Generator(device=self.device)
        g.manual_seed(_stream_seed(self.seed, name))
        if s.kind == "int_table":
            return torch.randint(0, 2 ** 15, tuple(s.shape), generator=g, device=self.device, dtype=torch.int32)
        t = torch.empty(tuple(s.shape), dtype=torch.float32, device=self.device)
        t.normal_(0.0, s.std, generator=g)
        if s.init == "one_plus_normal":
            t += 1.0
        return t.to(self.dtype(name))


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
