"""The one registry from an architecture's name to its configuration and model.

A name is accepted here and nowhere else: config.json's `architectures[0]`
(a class name such as "Qwen3ForCausalLM") or its `model_type` ("qwen3") selects
an entry; the entry's configuration class reads config.json strictly, and its
builder composes a `Model` from parameterised parts.  The reference keeps the
same single table (src/model/arch/registry.hpp:25-60).

Adding an architecture is one `register_architecture` call with
  * a `ModelConfig` subclass (`from_dict` / `to_dict`), and
  * `build(config) -> llmx_b200.models.Model`.
Nothing else in the package names an architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Tuple, Type

from .config.base import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: Type[ModelConfig]
    build: Callable[[ModelConfig], Any]


_BY_NAME: Dict[str, ArchitectureEntry] = {}


def register_architecture(names: Iterable[str], config_cls: Type[ModelConfig],
                          build: Callable[[ModelConfig], Any], *, replace: bool = False) -> ArchitectureEntry:
    names = list(names)
    if not names:
        raise ValueError("an architecture needs at least one name")
    entry = ArchitectureEntry(names[0], config_cls, build)
    for n in names:
        if n in _BY_NAME and not replace:
            raise ValueError(f"architecture name {n!r} is already registered")
        _BY_NAME[n] = entry
    return entry


def unregister_architecture(names: Iterable[str]) -> None:
    for n in names:
        _BY_NAME.pop(n, None)


def registered_names() -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_BY_NAME))


def architecture_of(raw_config: Dict[str, Any]) -> ArchitectureEntry:
    """The entry config.json names, by `architectures[0]` first, then `model_type`."""
    _ensure_builtin()
    archs = raw_config.get("architectures")
    tried = []
    if isinstance(archs, list) and len(archs) == 1 and isinstance(archs[0], str):
        tried.append(archs[0])
        if archs[0] in _BY_NAME:
            return _BY_NAME[archs[0]]
    mt = raw_config.get("model_type")
    if isinstance(mt, str):
        tried.append(mt)
        if mt in _BY_NAME:
            return _BY_NAME[mt]
    raise ConfigError(
        f"config.json names no architecture this engine has (tried {tried or 'nothing'}; "
        f"registered: {', '.join(sorted(_BY_NAME))})")


def config_from_dir(model_dir: str) -> Tuple[ArchitectureEntry, ModelConfig]:
    raw = read_config_json(model_dir)
    entry = architecture_of(raw)
    return entry, entry.config_cls.from_dict(raw)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from .models import qwen3 as _qwen3  # noqa: F401  (registers itself)
