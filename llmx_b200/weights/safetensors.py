"""Reading and writing safetensors files, by tensor name.

The format: 8 bytes little-endian header length N, N bytes of JSON mapping a
tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (plus an
optional "__metadata__" object of strings), then the data, whose offsets are
relative to the end of the header.  Shapes are outermost-first (row-major).

A model folder holds either one `model.safetensors` or a
`model.safetensors.index.json` whose `weight_map` names the file of every
tensor.  File-level refusals follow the reference's reader
(src/format/safetensors.hpp:20-25, :66-138, index file :141-170): an oversized
or truncated header, a header that is not an object, a repeated name, an entry
with other keys than the three, offsets that do not span the shape, gaps or
overlaps between tensors, data that does not end at the end of the file, and an
index that points outside the folder or disagrees with the files.

Tensors are memory-mapped and returned as CPU torch tensors that alias the
mapping (no copy until they are moved to the device).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch


class SafetensorsError(ValueError):
    """A safetensors file or folder that cannot be read."""


_DTYPES: Dict[str, Tuple[torch.dtype, int]] = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}

MAX_HEADER_BYTES = 100 * 1024 * 1024
MAX_RANK = 5


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int          # byte offsets in the file (absolute)
    end: int
    path: str


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise SafetensorsError(f"header repeats the key {k!r}")
        seen[k] = v
    return seen


def read_header(path: str) -> Tuple[Dict[str, TensorEntry], Dict[str, str]]:
    """Parse and validate one file's header; returns (entries by name, metadata)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: header of {n} bytes exceeds {MAX_HEADER_BYTES}")
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header runs past the end of the file")
        text = f.read(n)
    try:
        raw = json.loads(text.decode("utf-8"), object_pairs_hook=_no_duplicates)
    except SafetensorsError as e:
        raise SafetensorsError(f"{path}: {e}") from None
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
    if not isinstance(raw, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    meta = raw.pop("__metadata__", {}) or {}
    if not isinstance(meta, dict) or any(not isinstance(v, str) for v in meta.values()):
        raise SafetensorsError(f"{path}: __metadata__ must map strings to strings")
    base = 8 + n
    entries: Dict[str, TensorEntry] = {}
    for name, e in raw.items():
        if not isinstance(e, dict) or set(e) != {"dtype", "shape", "data_offsets"}:
            raise SafetensorsError(f"{path}: tensor {name!r} must have exactly dtype, shape and data_offsets")
        if e["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {e['dtype']!r}")
        dtype, width = _DTYPES[e["dtype"]]
        shape = e["shape"]
        if (not isinstance(shape, list) or len(shape) > MAX_RANK
                or any(not isinstance(d, int) or isinstance(d, bool) or d < 0 for d in shape)):
            raise SafetensorsError(f"{path}: tensor {name!r} has an invalid shape {shape!r}")
        off = e["data_offsets"]
        if (not isinstance(off, list) or len(off) != 2
                or any(not isinstance(o, int) or isinstance(o, bool) or o < 0 for o in off) or off[0] > off[1]):
            raise SafetensorsError(f"{path}: tensor {name!r} has invalid data_offsets {off!r}")
        count = 1
        for d in shape:
            count *= d
        if off[1] - off[0] != count * width:
            raise SafetensorsError(
                f"{path}: tensor {name!r}: offsets span {off[1] - off[0]} bytes, shape {shape} of {e['dtype']} needs {count * width}")
        if off[0] % width:
            raise SafetensorsError(f"{path}: tensor {name!r}: data is not aligned to its element size")
        entries[name] = TensorEntry(name, dtype, tuple(shape), base + off[0], base + off[1], path)
    # No gaps, no overlaps, and the data ends where the file ends.
    at = base
    for e in sorted(entries.values(), key=lambda t: (t.begin, t.end)):
        if e.begin != at:
            what = "overlaps the tensor before it" if e.begin < at else "leaves a gap before it"
            raise SafetensorsError(f"{path}: tensor {e.name!r} {what}")
        at = e.end
    if at != size:
        raise SafetensorsError(f"{path}: tensor data ends at byte {at}, the file at {size}")
    return entries, meta


class SafetensorsFile:
    """One memory-mapped file; `tensor(name)` aliases the mapping."""

    def __init__(self, path: str):
        self.path = path
        self.entries, self.metadata = read_header(path)
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(path) else None

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        count = 1
        for d in e.shape:
            count *= d
        if count == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; the tensor is never written
            t = torch.frombuffer(self._map, dtype=e.dtype, count=count, offset=e.begin)
        return t.view(e.shape)

    def close(self) -> None:
        # Tensors handed out alias the mapping; it is closed only if none does.
        try:
            if self._map is not None:
                self._map.close()
        except BufferError:
            pass
        self._file.close()


class TensorDirectory:
    """All tensors of a model folder, by name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self.files: List[SafetensorsFile] = []
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        if os.path.exists(index):
            self._read_index(index)
        elif os.path.exists(single):
            self._add(SafetensorsFile(single))
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def _add(self, f: SafetensorsFile) -> None:
        self.files.append(f)
        for name, e in f.entries.items():
            if name in self.entries:
                raise SafetensorsError(f"tensor {name!r} is in both {self.entries[name].path} and {f.path}")
            self.entries[name] = e
            self._owner[name] = f

    def _read_index(self, index: str) -> None:
        try:
            with open(index, "r", encoding="utf-8") as fh:
                raw = json.load(fh, object_pairs_hook=_no_duplicates)
        except (json.JSONDecodeError, SafetensorsError) as e:
            raise SafetensorsError(f"{index}: {e}") from None
        wm = raw.get("weight_map") if isinstance(raw, dict) else None
        if not isinstance(wm, dict) or any(not isinstance(v, str) for v in wm.values()):
            raise SafetensorsError(f"{index}: weight_map must map tensor names to file names")
        by_file: Dict[str, List[str]] = {}
        for name, fname in wm.items():
            if os.path.basename(fname) != fname or fname in ("", ".", ".."):
                raise SafetensorsError(f"{index}: {fname!r} names a path outside the model folder")
            by_file.setdefault(fname, []).append(name)
        for fname in sorted(by_file):
            f = SafetensorsFile(os.path.join(self.model_dir, fname))
            named, held = set(by_file[fname]), set(f.entries)
            if named != held:
                diff = sorted(named ^ held)
                raise SafetensorsError(f"{index}: weight_map and {fname} disagree on {', '.join(diff[:8])}")
            self._add(f)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name].dtype

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write CPU tensors to `path` in name order, contiguous, no gaps."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    at = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be written")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + nbytes]}
        at += nbytes
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                flat = t.reshape(-1)
                raw = flat.numpy() if t.dtype == torch.bool else flat.view(torch.uint8).numpy()
                f.write(memoryview(raw))
    os.replace(tmp, path)
