"""Typed configurations read from config.json."""
from .base import ConfigError, ModelConfig, Rule, apply_rules, read_config_json
from .qwen3 import Qwen3Config, YarnScaling

__all__ = ["ConfigError", "ModelConfig", "Rule", "apply_rules", "read_config_json", "Qwen3Config", "YarnScaling"]
