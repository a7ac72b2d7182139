from .base import ConfigError, Field, load_json, read_fields
from .gpt2 import ACT_ERF, ACT_TANH, GPT2Config
from .presets import load_preset, preset_json, preset_names, preset_random_options
from .registry import (Architecture, architectures, get_architecture, load_config,
                       register_architecture, resolve_architecture)

__all__ = [
    "ConfigError", "Field", "load_json", "read_fields", "GPT2Config", "ACT_TANH", "ACT_ERF",
    "Architecture", "architectures", "get_architecture", "load_config",
    "register_architecture", "resolve_architecture", "load_preset", "preset_json",
    "preset_names", "preset_random_options",
]
