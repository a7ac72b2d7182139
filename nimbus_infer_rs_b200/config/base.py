"""Typed reading of ``config.json`` values.

A configuration class declares its fields once (name, type, accepted key
spellings, default, check) and :func:`read_fields` turns a parsed JSON object into
keyword arguments, raising one :class:`ConfigError` that names every bad key.

The reference reads each key with a typed getter and keeps the default when a key
is absent or ``null`` (src/config.rs:69-133); unknown keys are ignored there and
here.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Sequence


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the chosen architecture."""


@dataclass(frozen=True)
class Field:
    """One typed entry of a configuration.

    ``keys`` lists the accepted spellings in order of precedence; ``kind`` is one of
    ``int``, ``float``, ``bool``, ``str``; ``choices`` maps accepted strings to the
    canonical value (for enums).
    """

    name: str
    kind: type
    keys: Sequence[str]
    default: Any = None
    required: bool = False
    choices: dict[str, Any] | None = None
    check: Callable[[Any], str | None] | None = None


def _positive(v) -> str | None:
    return None if v > 0 else "must be positive"


def _non_negative(v) -> str | None:
    return None if v >= 0 else "must not be negative"


positive = _positive
non_negative = _non_negative


def _coerce(field: Field, key: str, raw: Any) -> Any:
    kind = field.kind
    if kind is bool:
        if isinstance(raw, bool):
            return raw
        raise ConfigError(f"{key}: expected true/false, got {raw!r}")
    if kind is int:
        if isinstance(raw, bool) or not isinstance(raw, (int, float)):
            raise ConfigError(f"{key}: expected an integer, got {raw!r}")
        if float(raw) != int(raw):
            raise ConfigError(f"{key}: expected an integer, got {raw!r}")
        return int(raw)
    if kind is float:
        if isinstance(raw, bool) or not isinstance(raw, (int, float)):
            raise ConfigError(f"{key}: expected a number, got {raw!r}")
        return float(raw)
    if kind is str:
        if not isinstance(raw, str):
            raise ConfigError(f"{key}: expected a string, got {raw!r}")
        if field.choices is not None:
            if raw not in field.choices:
                raise ConfigError(
                    f"{key}: unknown value {raw!r} (accepted: {sorted(field.choices)})"
                )
            return field.choices[raw]
        return raw
    raise TypeError(f"field {field.name}: unsupported kind {kind}")


def read_fields(obj: dict, fields: Sequence[Field]) -> tuple[dict, dict]:
    """Return ``(values, used_key)``: the typed values and, per field, the key
    spelling that supplied it (``None`` when the default was taken)."""
    if not isinstance(obj, dict):
        raise ConfigError("config.json must hold a JSON object")
    values: dict[str, Any] = {}
    used: dict[str, str | None] = {}
    problems: list[str] = []
    for f in fields:
        chosen = None
        for key in f.keys:
            if key in obj and obj[key] is not None:
                chosen = key
                break
        used[f.name] = chosen
        if chosen is None:
            if f.required:
                problems.append(f"{'/'.join(f.keys)}: missing")
            values[f.name] = f.default
            continue
        try:
            v = _coerce(f, chosen, obj[chosen])
            if f.check is not None:
                msg = f.check(v)
                if msg:
                    raise ConfigError(f"{chosen}: {msg} (got {v!r})")
            values[f.name] = v
        except ConfigError as e:
            problems.append(str(e))
            values[f.name] = f.default
    if problems:
        raise ConfigError("bad config.json: " + "; ".join(problems))
    return values, used


def load_json(path: str | Path) -> dict:
    path = Path(path)
    try:
        text = path.read_text(encoding="utf-8")
    except OSError as e:
        raise ConfigError(f"reading {path}: {e}") from e
    try:
        obj = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return obj
