"""One registry from an architecture's name to everything that builds its model.

An :class:`Architecture` bundles the typed configuration class, the function that
turns a configuration into a :class:`~nimbus_infer_rs_b200.engine.spec.ModelSpec`
(which parts, layer by layer, in which order), and the function that says where each
parameter comes from in a weight file.  Nothing else in the package names a model.

The reference has no registry: one ``Model`` struct is switched by three enums
(src/config.rs:27-43, src/model.rs:171-181).  A config.json in the reference's style
is therefore recognised by those enums; other styles by ``model_type`` or
``architectures``.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .base import ConfigError, load_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    build_spec: Callable[[Any], Any]          # config -> ModelSpec
    weight_plan: Callable[[Any, Any, set], Any]  # (config, spec, names in file) -> WeightPlan
    aliases: tuple[str, ...] = ()
    # (config, seed, **options) -> {tensor name: CPU tensor}: the random-weights mode
    random_tensors: Callable[..., dict] | None = None
    # Called with the raw config.json object; True if this architecture claims it when
    # no explicit name key is present.
    recognises: Callable[[dict], bool] | None = None


_ARCHITECTURES: dict[str, Architecture] = {}
_ALIASES: dict[str, str] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    for a in (arch.name, *arch.aliases):
        _ALIASES[a.lower()] = arch.name
    return arch


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    key = _ALIASES.get(str(name).lower())
    if key is None:
        raise ConfigError(
            f"architecture not supported: {name!r} (registered: {architectures()})")
    return _ARCHITECTURES[key]


def resolve_architecture(obj: dict) -> Architecture:
    """Choose the architecture that a parsed config.json describes."""
    for key in ("architecture", "model_type"):
        v = obj.get(key)
        if isinstance(v, str):
            return get_architecture(v)
    v = obj.get("architectures")
    if isinstance(v, list) and v and isinstance(v[0], str):
        return get_architecture(v[0])
    claimed = [a for a in _ARCHITECTURES.values() if a.recognises and a.recognises(obj)]
    if len(claimed) == 1:
        return claimed[0]
    if not claimed:
        raise ConfigError(
            "architecture not supported: config.json names no registered architecture "
            f"(norm={obj.get('norm')!r}, activation={obj.get('activation')!r}, "
            f"pos_encoding={obj.get('pos_encoding')!r}; registered: {architectures()})")
    raise ConfigError(
        "config.json is ambiguous between architectures "
        f"{sorted(a.name for a in claimed)}; add a 'model_type' key")


def load_config(model_dir: str | Path):
    """Read ``config.json`` of a model folder → ``(architecture, typed config)``."""
    obj = load_json(Path(model_dir) / "config.json")
    arch = resolve_architecture(obj)
    return arch, arch.config_cls.from_json(obj)
