"""Random-weights mode: write a model folder (config.json + model.safetensors) from a
configuration and a seed.

Which tensors a model has, under which names and with which shapes, is the architecture's
knowledge: its registry entry supplies ``random_tensors(config, seed, **options)``.  This file
only writes what that function returns, next to the configuration.

The reference's fixture was made this way by its sibling engine
(benchmarks/cross_engine.py:43-64: ``Engine.random(config, seed=42)``).
"""
from __future__ import annotations

import json
from pathlib import Path

from ..config.registry import get_architecture
from .safetensors_io import write_safetensors


def write_random_model(model_dir: str | Path, cfg, seed: int, **kw) -> Path:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir`` for any registered
    architecture's configuration."""
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    arch = get_architecture(cfg.architecture)
    if arch.random_tensors is None:
        raise ValueError(f"architecture {arch.name!r} has no random-weights mode")
    tensors = arch.random_tensors(cfg, seed, **kw)
    (d / "config.json").write_text(json.dumps(cfg.to_json(), indent=2) + "\n")
    write_safetensors(d / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return d
