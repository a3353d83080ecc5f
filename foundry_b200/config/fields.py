"""Typed reads of a decoded config.json: a key that must be there with a value of
the right kind, with the place named in the error."""
from __future__ import annotations

from typing import Any, Mapping

from . import errors


def need(doc: Mapping[str, Any], key: str, kind, where: str):
    if key not in doc or doc[key] is None:
        raise errors.ConfigJson(f"{where}: key {key!r} is missing")
    value = doc[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if not isinstance(value, kind) or isinstance(value, bool) and kind is not bool:
        raise errors.ConfigJson(f"{where}: key {key!r} should be {kind.__name__}, found {value!r}")
    return value


def positive(doc, key, where) -> int:
    value = need(doc, key, int, where)
    if value <= 0:
        raise errors.ConfigJson(f"{where}: {key} = {value} must be positive")
    return value
