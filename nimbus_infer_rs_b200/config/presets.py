"""Named model sizes for the random-weights mode: ``gpt2`` (124M, the reference's defaults,
src/config.rs:45-66), ``gpt2-medium`` (355M), ``gpt2-xl`` (1.5B) and the two test sizes
``tiny-a`` and ``tiny-b``.

A preset is a ``config.json`` object kept as a file under ``presets/`` (no size stands in
code), read through the same registry and typed parser as a model folder's config.  Next to
the configuration keys a preset may hold ``random_weights``: the spread of the random values
(``std``, ``bias_std``, ``gamma_jitter``, ``beta_std``) that the random-weights mode uses for
it unless the caller says otherwise.
"""
from __future__ import annotations

from pathlib import Path

from .base import ConfigError, load_json
from .registry import resolve_architecture

PRESET_DIR = Path(__file__).resolve().parent / "presets"
_EXTRA_KEYS = ("_about", "random_weights")


def preset_names() -> list[str]:
    return sorted(p.stem for p in PRESET_DIR.glob("*.json"))


def preset_json(name: str) -> dict:
    """The preset's config.json object (without the keys that are not configuration)."""
    obj = _load(name)
    return {k: v for k, v in obj.items() if k not in _EXTRA_KEYS}


def preset_random_options(name: str) -> dict:
    """Keyword arguments for the architecture's random tensors (``std`` and the like)."""
    opts = _load(name).get("random_weights") or {}
    if not isinstance(opts, dict):
        raise ConfigError(f"preset {name!r}: random_weights must be an object")
    return dict(opts)


def load_preset(name: str):
    """``(architecture, typed config, random-weight options)`` of a preset."""
    obj = preset_json(name)
    arch = resolve_architecture(obj)
    return arch, arch.config_cls.from_json(obj), preset_random_options(name)


def _load(name: str) -> dict:
    key = str(name).strip().lower()
    path = PRESET_DIR / f"{key}.json"
    if "/" in key or "\\" in key or not path.is_file():
        raise ConfigError(f"no preset named {name!r} (have: {', '.join(preset_names())})")
    return load_json(path)
