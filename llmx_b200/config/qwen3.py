"""Typed configuration of the dense Qwen3 architecture, read from config.json.

Keys, defaults and refusals follow the reference's table for this
architecture (src/model/arch/qwen3.hpp:107-139) and its checks
(src/model/arch/qwen3.hpp:47-60, :63-104; rope_scaling in
src/model/arch/hf_config.hpp:125-155 and src/model/rope.hpp:105-146).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict, replace
from typing import Any, Dict, Optional

from .base import ConfigError, ModelConfig, Rule, apply_rules, _is_int

_DTYPES = ("bfloat16", "float16", "float32")

_TABLE: Dict[str, Rule] = {
    "num_hidden_layers": Rule("integer", required=True),
    "hidden_size": Rule("integer", required=True),
    "intermediate_size": Rule("integer", required=True),
    "num_attention_heads": Rule("integer", required=True),
    "num_key_value_heads": Rule("integer"),
    "head_dim": Rule("integer"),
    "max_position_embeddings": Rule("integer"),
    "rope_theta": Rule("real"),
    "rms_norm_eps": Rule("real"),
    "vocab_size": Rule("integer", required=True),
    "tie_word_embeddings": Rule("boolean"),
    "rope_scaling": Rule("keep"),
    # Checked, then without effect on the forward pass.
    "attention_bias": Rule("check", allowed=(False,)),
    "hidden_act": Rule("check", allowed=("silu",)),
    "use_sliding_window": Rule("check", allowed=(False,)),
    "layer_types": Rule("each", allowed=("full_attention",)),
    "torch_dtype": Rule("check", allowed=_DTYPES),
    "dtype": Rule("check", allowed=_DTYPES),
    "architectures": Rule("check", allowed=(["Qwen3ForCausalLM"],)),
    "model_type": Rule("check", allowed=("qwen3",)),
    # Token ids: used by generation (a reply ends at eos), not by the model.
    "bos_token_id": Rule("keep"),
    "eos_token_id": Rule("keep"),
    "pad_token_id": Rule("keep"),
    # Accepted and ignored.
    "attention_dropout": Rule("check"),
    "initializer_range": Rule("check"),
    "max_window_layers": Rule("check"),
    "sliding_window": Rule("check"),
    "transformers_version": Rule("check"),
    "use_cache": Rule("check"),
    "unsloth_fixed": Rule("check"),
}


@dataclass(frozen=True)
class YarnScaling:
    """YaRN rope scaling as config.json's rope_scaling object gives it."""
    factor: float
    original_max_position_embeddings: int
    beta_fast: float = 32.0
    beta_slow: float = 1.0

    @property
    def attention_factor(self) -> float:
        # 0.1 ln(factor) + 1 on cos and sin (src/model/rope.hpp:145).
        return float(0.1 * math.log(self.factor) + 1.0)


def _read_rope_scaling(value: Any, max_pos: int) -> Optional[YarnScaling]:
    if value is None:
        return None
    if not isinstance(value, dict):
        raise ConfigError("qwen3: rope_scaling is not an object or null")
    seen = set(value)
    kind = value.get("rope_type", value.get("type"))
    if "rope_type" not in seen and "type" not in seen:
        raise ConfigError("qwen3: rope_scaling gives no rope_type")
    for k in ("rope_type", "type"):
        if k in value and value[k] != "yarn":
            raise ConfigError(f"qwen3: rope_scaling.{k} = {value[k]!r} is not supported (\"yarn\")")
    for k in value:
        if k in ("attention_factor", "mscale", "mscale_all_dim"):
            raise ConfigError(f"qwen3: rope_scaling.{k} is not supported")
        if k not in ("rope_type", "type", "factor", "original_max_position_embeddings", "beta_fast", "beta_slow"):
            raise ConfigError(f"qwen3: rope_scaling.{k} is not a key this engine reads")
    if "factor" not in value:
        raise ConfigError("qwen3: rope_scaling gives no factor")

    def real(k: str, default: float) -> float:
        v = value.get(k, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
            raise ConfigError(f"qwen3: rope_scaling.{k} must be a finite number, got {v!r}")
        return float(v)

    factor = real("factor", 1.0)
    if not factor > 1.0:
        raise ConfigError("qwen3: rope_scaling.factor must be above 1 for YaRN")
    orig = value.get("original_max_position_embeddings", max_pos)
    if not _is_int(orig) or orig < 1:
        raise ConfigError(f"qwen3: rope_scaling.original_max_position_embeddings must be a positive integer, got {orig!r}")
    fast, slow = real("beta_fast", 32.0), real("beta_slow", 1.0)
    if not fast > slow:
        raise ConfigError("qwen3: rope_scaling.beta_fast must be above beta_slow")
    assert kind == "yarn"
    return YarnScaling(factor, int(orig), fast, slow)


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int = 4096
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    rope_scaling: Optional[YarnScaling] = None
    bos_token_id: Any = None
    eos_token_id: Any = None
    pad_token_id: Any = None

    model_type = "qwen3"
    class_name = "Qwen3ForCausalLM"

    def __post_init__(self) -> None:
        h, g, d = self.num_attention_heads, self.num_key_value_heads, self.head_dim
        if h % g:
            raise ConfigError("qwen3: head count must be divisible by KV head count")
        if d <= 0 or d % 2:
            raise ConfigError("qwen3: invalid attention projection dimensions (head_dim must be even and positive)")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError("qwen3: invalid rope base")
        if not self.rms_norm_eps >= 0:
            raise ConfigError("qwen3: rms_norm_eps must not be negative")

    # -- derived widths -----------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def eos_ids(self) -> tuple:
        e = self.eos_token_id
        if e is None:
            return ()
        if isinstance(e, list):
            return tuple(int(x) for x in e)
        return (int(e),)

    def with_yarn(self, factor: float, original: Optional[int] = None) -> "Qwen3Config":
        """This configuration with its rope scaled by YaRN at `factor` (what --yarn asks, src/model/rope.hpp:131-146):
        over `original` positions if given (at most the model's context), else over the original length the file
        declares, else over the file's context; the context becomes floor(factor x original).  The file's beta_fast
        and beta_slow are kept when it declares YaRN itself."""
        if not (isinstance(factor, (int, float)) and math.isfinite(factor) and factor > 1):
            raise ConfigError("qwen3: --yarn must be a finite factor above 1")
        declared = self.rope_scaling
        if original is not None:
            if not _is_int(original) or original < 1 or original > self.max_position_embeddings:
                raise ConfigError(f"qwen3: --yarn-original-ctx {original} is past the model's context of "
                                  f"{self.max_position_embeddings}")
            base = int(original)
        else:
            base = declared.original_max_position_embeddings if declared else self.max_position_embeddings
        context = math.floor(float(factor) * base)
        if context > 2 ** 31 - 1:
            raise ConfigError(f"qwen3: --yarn {factor} over {base} is past the context limit")
        scaling = YarnScaling(float(factor), base, declared.beta_fast if declared else 32.0,
                              declared.beta_slow if declared else 1.0)
        return replace(self, rope_scaling=scaling, max_position_embeddings=int(context))

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        got = apply_rules(raw, _TABLE, "qwen3")
        if "architectures" in raw and raw["architectures"] != ["Qwen3ForCausalLM"]:
            raise ConfigError("qwen3: architectures must be [\"Qwen3ForCausalLM\"]")
        h = got["num_attention_heads"]
        got.setdefault("num_key_value_heads", h)
        if "head_dim" not in got:
            if got["hidden_size"] % h:
                raise ConfigError("qwen3: embedding width does not determine an integral head width")
            got["head_dim"] = got["hidden_size"] // h
        max_pos = got.get("max_position_embeddings", 4096)
        got["rope_scaling"] = _read_rope_scaling(got.get("rope_scaling"), max_pos)
        got.pop("layer_types", None)
        for k in ("bos_token_id", "eos_token_id", "pad_token_id"):
            v = got.get(k)
            ok = v is None or _is_int(v) or (isinstance(v, list) and all(_is_int(x) for x in v))
            if not ok:
                raise ConfigError(f"qwen3: {k} must be an integer, a list of integers or null, got {v!r}")
        return cls(**got)

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        rs = d.pop("rope_scaling")
        d["rope_scaling"] = None if rs is None else {"rope_type": "yarn", **rs}
        d = {k: v for k, v in d.items() if v is not None or k == "rope_scaling"}
        d["architectures"] = [self.class_name]
        d["model_type"] = self.model_type
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["use_sliding_window"] = False
        return d
