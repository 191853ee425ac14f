"""Typed configurations read from config.json."""
from .base import ConfigError, ModelConfig, Rule, apply_rules, read_config_json
from .qwen3 import Qwen3Config, YarnScaling
from .buzetar import BuzetarConfig
from .kisepel import KisepelConfig
from .zamizen import ZamizenConfig
from .nomutar import NomutarConfig

__all__ = ["ConfigError", "ModelConfig", "Rule", "apply_rules", "read_config_json", "Qwen3Config", "YarnScaling", "BuzetarConfig", "KisepelConfig", "ZamizenConfig", "NomutarConfig"]
