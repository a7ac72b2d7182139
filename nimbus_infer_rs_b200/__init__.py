"""A small GPT-2 generation library for one NVIDIA B200 (sm_100a): from a model folder
(config.json + safetensors) to generated tokens, through hand-written CUDA kernels only.

    from nimbus_infer_rs_b200 import Engine, SamplingParams
    engine = Engine.load("model_dir", dtype="bfloat16")
    new_ids = engine.generate([[5, 17, 3]], SamplingParams(max_new_tokens=8, temperature=0.0))
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, GPT2Config, get_architecture, load_config, register_architecture
from .engine import Engine, LayerSpec, ModelSpec
from .parts import PartSpec, register_part
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["Engine", "SamplingParams", "GPT2Config", "ConfigError", "WeightError", "ModelSpec",
           "LayerSpec", "PartSpec", "register_part", "register_architecture",
           "get_architecture", "load_config", "write_random_model"]
