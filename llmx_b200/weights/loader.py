"""Weights by tensor name: checked against the model's expectations, then handed to its parts.

A *source* is anything with `names()`, `shape(name)`, `dtype(name)` and
`tensor(name)`: a folder of safetensors files (`TensorDirectory`) or the seeded
random generator (`RandomSource`).  `check_tensors` compares a source with the
model's `tensor_specs()` and raises one `WeightError` naming every missing,
unexpected and ill-shaped tensor (the reference refuses them one at a time:
src/model/arch/hf_config.hpp:317-336, src/model/weights.hpp:77-92,
src/model/architecture.hpp:73-86).

Storage types are kept: a bfloat16 tensor stays bfloat16, a 32-bit tensor stays
32-bit, integer tables become int32.  What a *part* then computes with is the
part's business (`Part.load`): matrices are cast to the compute type of the
path, norm vectors are always widened to 32-bit
(src/inference/directory.hpp:69-71, src/inference/load.hpp:470-494).
"""
from __future__ import annotations

from typing import Dict, Iterable, Mapping, Optional, Set

import torch

from .spec import TensorSpec, WeightError

_FLOATS = (torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_tensors(specs: Mapping[str, TensorSpec], source, where: str,
                  ignorable: Iterable[str] = ()) -> None:
    """Raise one WeightError if `source` does not hold exactly what `specs` asks.

    `ignorable` names tensors that may be present without being read (a tied
    model's stored lm_head, which the reference drops: hf_config.hpp:300-335).
    """
    have = set(source.names())
    ignorable = set(ignorable)
    missing = sorted(n for n, s in specs.items() if n not in have and not s.optional)
    unexpected = sorted(n for n in have if n not in specs and n not in ignorable)
    wrong = []
    for n, s in specs.items():
        if n not in have:
            continue
        shape, dtype = tuple(source.shape(n)), source.dtype(n)
        if shape != tuple(s.shape):
            wrong.append((n, f"shape {list(shape)}, expected {list(s.shape)}"))
        elif s.kind == "int_table" and dtype not in _INTS:
            wrong.append((n, f"type {dtype}, expected an integer type"))
        elif s.kind != "int_table" and dtype not in _FLOATS:
            wrong.append((n, f"type {dtype}, expected float32, float16 or bfloat16"))
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)


def stored(source, name: str, spec: TensorSpec, device) -> torch.Tensor:
    """The tensor on `device` in its storage type (int tables as int32, float16 widened to float32)."""
    t = source.tensor(name)
    if spec.kind == "int_table":
        return t.to(device=device, dtype=torch.int32)
    if t.dtype == torch.float16:
        # float16 files are accepted; every float16 value is exact in float32.
        return t.to(device=device, dtype=torch.float32)
    return t.to(device=device)
