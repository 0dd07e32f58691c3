"""What a model expects of its tensors, and the one error that says what is wrong."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part reads.

    kind: "matrix"  [out, in] row-major, each output row contiguous (a weight of a product)
          "table"   [rows, width] gathered by id (an embedding)
          "vector"  a norm's weight; held in 32-bit on the device whatever the file stores
          "int_table" integer table, held as int32
    init: how the random-weights mode fills it: "normal" (N(0, std)) or "one_plus_normal" (1 + N(0, std)).
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    optional: bool = False
    init: str = "normal"
    std: float = 0.02


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model.

    One error lists everything at once: tensors the model needs and the files
    lack, tensors the files hold and the model does not know, and tensors of
    the wrong shape or type.
    """

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong: Sequence[Tuple[str, str]]):
        self.missing: List[str] = list(missing)
        self.unexpected: List[str] = list(unexpected)
        self.wrong: List[Tuple[str, str]] = list(wrong)
        lines = [f"{where}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or type ({len(self.wrong)}): " +
                         "; ".join(f"{n}: {why}" for n, why in self.wrong))
        super().__init__("\n".join(lines))
