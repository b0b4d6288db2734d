"""Strict reading of a model's ``config.json``.

The reference reads flat scalar keys only and refuses a file that repeats a
key (src/alofa/model/config.mojo:46-100): a duplicated key means two tools
disagree about the model, and picking either silently is wrong.  The same rule
is kept here; nested values are passed through for the few keys that are
lists (``architectures``)."""
from __future__ import annotations

import json
from pathlib import Path

from ..errors import AlofaError


def _no_duplicates(pairs):
    seen = {}
    for key, value in pairs:
        if key in seen:
            raise AlofaError("parse", "config.json repeats a key", f"key={key}")
        seen[key] = value
    return seen


def read_json_object(path) -> dict:
    """The top-level object of a JSON file, refusing duplicate keys."""
    path = Path(path)
    try:
        text = path.read_text()
    except OSError as err:
        raise AlofaError("io", "cannot read config file", f"config={path}: {err}") from err
    try:
        obj = json.loads(text, object_pairs_hook=_no_duplicates)
    except json.JSONDecodeError as err:
        raise AlofaError("parse", "config file is not valid JSON", f"config={path}: {err}") from err
    if not isinstance(obj, dict):
        raise AlofaError("parse", "config file must hold one JSON object", f"config={path}")
    return obj


class Keys:
    """Typed access to the keys of one config object; every failure names the
    key and the file."""

    def __init__(self, obj: dict, origin: str):
        self.obj = obj
        self.origin = origin

    def _missing(self, key):
        return AlofaError("parse", "config key is missing", f"key={key} config={self.origin}")

    def has(self, key: str) -> bool:
        return key in self.obj and self.obj[key] is not None

    def integer(self, key: str, default=None) -> int:
        if not self.has(key):
            if default is None:
                raise self._missing(key)
            return default
        value = self.obj[key]
        if isinstance(value, bool) or not isinstance(value, int):
            raise AlofaError("parse", "config key must be an integer", f"{key}={value!r} config={self.origin}")
        return value

    def number(self, key: str, default=None) -> float:
        if not self.has(key):
            if default is None:
                raise self._missing(key)
            return default
        value = self.obj[key]
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise AlofaError("parse", "config key must be a number", f"{key}={value!r} config={self.origin}")
        return float(value)

    def boolean(self, key: str, default=None) -> bool:
        if not self.has(key):
            if default is None:
                raise self._missing(key)
            return default
        value = self.obj[key]
        if not isinstance(value, bool):
            raise AlofaError("parse", "config key must be true or false", f"{key}={value!r} config={self.origin}")
        return value

    def string(self, key: str, default=None) -> str:
        if not self.has(key):
            if default is None:
                raise self._missing(key)
            return default
        value = self.obj[key]
        if not isinstance(value, str):
            raise AlofaError("parse", "config key must be a string", f"{key}={value!r} config={self.origin}")
        return value
