"""Strict reading of a model folder's config.json.

An architecture declares one table of the keys it understands.  Every key of
config.json must be in the table; a key outside it is refused by name, so a
checkpoint of one architecture is never read as another.  This mirrors the
strict key table of the reference (src/model/arch/hf_config.hpp:23-77, applied
at :263-373) without sharing its representation: here a rule is a small object
that validates and converts one JSON value.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Optional, Sequence


class ConfigError(ValueError):
    """config.json cannot be read as the architecture it names."""


@dataclass(frozen=True)
class Rule:
    """How one config.json key is read.

    kind:
      "integer"  a JSON integer >= `minimum` (no floats, no booleans)
      "real"     a finite JSON number
      "boolean"  true or false
      "check"    the value must be one of `allowed` (compared as JSON values);
                 with `allowed` None any value passes; never stored
      "each"     a list whose every element must be one of `allowed`
      "null"     must be null (used for options this engine refuses otherwise)
      "keep"     stored as it stands (ids used by generation, not by the model)
    """
    kind: str
    field: Optional[str] = None
    allowed: Optional[Sequence[Any]] = None
    minimum: int = 1
    required: bool = False


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def apply_rules(raw: Dict[str, Any], table: Dict[str, Rule], where: str) -> Dict[str, Any]:
    """Validate `raw` against `table`; return {field: value} for the stored keys."""
    out: Dict[str, Any] = {}
    unknown = sorted(k for k in raw if k not in table)
    if unknown:
        raise ConfigError(f"{where}: unknown config.json key(s): {', '.join(unknown)}")
    missing = sorted(k for k, r in table.items() if r.required and k not in raw)
    if missing:
        raise ConfigError(f"{where}: missing config.json key(s): {', '.join(missing)}")
    for key, value in raw.items():
        rule = table[key]
        if rule.kind == "integer":
            if not _is_int(value) or value < rule.minimum:
                raise ConfigError(f"{where}: {key} must be an integer >= {rule.minimum}, got {value!r}")
            out[rule.field or key] = int(value)
        elif rule.kind == "real":
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
                raise ConfigError(f"{where}: {key} must be a finite number, got {value!r}")
            out[rule.field or key] = float(value)
        elif rule.kind == "boolean":
            if not isinstance(value, bool):
                raise ConfigError(f"{where}: {key} must be true or false, got {value!r}")
            out[rule.field or key] = value
        elif rule.kind == "check":
            if rule.allowed is not None and not any(value == a and type(value) is type(a) for a in rule.allowed):
                raise ConfigError(f"{where}: {key} must be one of {list(rule.allowed)!r}, got {value!r}")
        elif rule.kind == "each":
            if not isinstance(value, list) or any(not any(v == a for a in rule.allowed or ()) for v in value):
                raise ConfigError(f"{where}: every entry of {key} must be one of {list(rule.allowed or ())!r}, got {value!r}")
            out[rule.field or key] = list(value)
        elif rule.kind == "null":
            if value is not None:
                raise ConfigError(f"{where}: {key} is not supported (must be null), got {value!r}")
        elif rule.kind == "keep":
            out[rule.field or key] = value
        else:  # pragma: no cover - a table error, not a user error
            raise AssertionError(f"bad rule kind {rule.kind}")
    return out


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{model_dir}: no config.json") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: config.json must hold an object")
    return raw


class ModelConfig:
    """Base of every architecture's typed configuration.

    A subclass is a dataclass holding the numbers config.json gives, built by
    `from_dict` through its rule table and written back by `to_dict` (the
    random-weights mode writes a model folder from a configuration).
    """

    model_type: str = ""
    class_name: str = ""

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":  # pragma: no cover - interface
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:  # pragma: no cover - interface
        raise NotImplementedError

    @classmethod
    def from_dir(cls, model_dir: str) -> "ModelConfig":
        return cls.from_dict(read_config_json(model_dir))
