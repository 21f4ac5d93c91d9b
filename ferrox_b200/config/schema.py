"""Typed reading of a model's ``config.json``.

A configuration class lists its keys once, as :class:`Key` rows (name in
``config.json``, Python type, default or *required*, an optional check).
:func:`read_keys` turns a JSON object into validated values and raises one
:class:`ConfigError` that names every offending key, in the manner of the
reference's ``LoadError::MissingHparam`` (crates/ferrox-models/src/loader.rs:38-65),
which names the hyper-parameter it could not find.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Optional, Sequence


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a typed configuration."""


class _Required:
    def __repr__(self) -> str:  # pragma: no cover - cosmetic
        return "REQUIRED"


REQUIRED = _Required()


@dataclass(frozen=True)
class Key:
    """One row of a configuration schema."""

    name: str
    kind: type  # int, float, bool, str, list; object = any JSON value
    default: Any = REQUIRED  # REQUIRED, a value, or a callable(values_so_far) -> value
    check: Optional[Callable[[Any], Optional[str]]] = None  # returns an error text or None
    nullable: bool = False


def positive(v) -> Optional[str]:
    return None if v > 0 else "must be > 0"


def non_negative(v) -> Optional[str]:
    return None if v >= 0 else "must be >= 0"


def _coerce(key: Key, raw: Any) -> Any:
    if raw is None:
        if key.nullable:
            return None
        raise TypeError("is null")
    if key.kind is bool:
        if isinstance(raw, bool):
            return raw
        raise TypeError(f"expected true/false, found {raw!r}")
    if key.kind is int:
        if isinstance(raw, bool) or not isinstance(raw, (int, float)):
            raise TypeError(f"expected an integer, found {raw!r}")
        if isinstance(raw, float):
            if raw != int(raw):
                raise TypeError(f"expected an integer, found {raw!r}")
            raw = int(raw)
        return raw
    if key.kind is float:
        if isinstance(raw, bool) or not isinstance(raw, (int, float)):
            raise TypeError(f"expected a number, found {raw!r}")
        return float(raw)
    if key.kind is str:
        if not isinstance(raw, str):
            raise TypeError(f"expected a string, found {raw!r}")
        return raw
    if key.kind is list:
        if not isinstance(raw, (list, tuple)):
            raise TypeError(f"expected a list, found {raw!r}")
        return list(raw)
    if key.kind is object:
        return raw
    raise TypeError(f"schema error: unsupported kind {key.kind}")


def read_keys(obj: dict, schema: Sequence[Key], where: str = "config.json", ignore=None) -> dict:
    """Validate ``obj`` against ``schema``; returns {name: value}.  ``ignore``: the keys of ``obj`` beside the
    schema's that do not concern inference (book-keeping of the checkpoint: its dtype, the library version that
    wrote it, training settings).  With it, a key that neither the schema nor ``ignore`` lists is an error: the
    engine refuses a configuration that asks for something it does not implement rather than compute something
    else (the reference refuses metadata it cannot honour, crates/ferrox-models/src/capability.rs:616-637,
    loader.rs:141-158).  ``ignore=None`` ignores every unlisted key."""
    values: dict = {}
    problems: list[str] = []
    if ignore is not None:
        known = {k.name for k in schema} | set(ignore)
        for name in obj:
            if name not in known:
                problems.append(f"{name}: not a key this engine implements (refused rather than ignored)")
    for key in schema:
        if key.name in obj and not (obj[key.name] is None and not key.nullable and key.default is not REQUIRED):
            try:
                v = _coerce(key, obj[key.name])
            except TypeError as e:
                problems.append(f"{key.name}: {e}")
                continue
        elif key.default is REQUIRED:
            problems.append(f"{key.name}: required key is missing")
            continue
        elif callable(key.default):
            try:
                v = key.default(values)
            except KeyError as e:  # default depends on a key that failed
                problems.append(f"{key.name}: cannot derive default (needs {e})")
                continue
        else:
            v = key.default
        if v is not None and key.check is not None:
            msg = key.check(v)
            if msg:
                problems.append(f"{key.name}={v!r}: {msg}")
                continue
        values[key.name] = v
    if problems:
        raise ConfigError(f"{where}: " + "; ".join(problems))
    return values


def load_json(path: str) -> dict:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            obj = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return obj
