"""One registry from an architecture's name to its model.

``config.json`` carries ``architectures: ["Qwen2ForCausalLM"]``; the first
name chooses a :class:`Architecture`, which knows how to read that
architecture's own config keys into a typed configuration and how to turn the
configuration into a :class:`~alofa_b200.config.spec.ModelSpec`.  The
reference constructs its one model directly (src/alofa/cli.mojo:553) and has
no registry; this one exists so that another architecture is one more entry
and no change to loader, cache, engine or command line."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from ..errors import AlofaError
from .json_reader import read_json_object

_ARCHITECTURES: dict = {}


@dataclass
class Architecture:
    """``read_config(obj, origin)`` -> typed config; ``build_spec(config)`` ->
    ModelSpec; ``to_json(config)`` -> dict for config.json."""

    name: str
    read_config: Callable
    build_spec: Callable
    to_json: Callable


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise AlofaError("invalid_argument", "architecture is already registered", f"name={arch.name}")
    _ARCHITECTURES[arch.name] = arch


def known_architectures() -> list:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise AlofaError("unsupported", "no model is registered for this architecture", f"name={name} known={known_architectures()}")
    return _ARCHITECTURES[name]


_plugins_loaded = False


def _ensure_builtin() -> None:
    """Importing the models package registers the built-in architectures.
    ``ALOFA_PLUGINS`` (comma-separated module names, importable from the
    Python path) names modules of the user's own that register further parts
    and architectures when imported: the command-line programs, which build
    nothing but what config.json names, find them this way."""
    global _plugins_loaded
    from .. import models  # noqa: F401

    if not _plugins_loaded:
        _plugins_loaded = True
        import importlib
        import os

        for name in filter(None, (m.strip() for m in os.environ.get("ALOFA_PLUGINS", "").split(","))):
            try:
                importlib.import_module(name)
            except ImportError as err:
                raise AlofaError("invalid_argument", "a module named in ALOFA_PLUGINS cannot be imported", f"module={name}: {err}") from err


def architecture_name_of(obj: dict, origin: str) -> str:
    names = obj.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise AlofaError("parse", "config.json must name its architecture in 'architectures'", f"config={origin}")
    return names[0]


def read_model_config(folder):
    """(architecture, typed config) of a model folder, chosen by config.json."""
    return read_model_config_file(Path(folder) / "config.json")


def read_model_config_file(path):
    """(architecture, typed config) of a config.json under any file name."""
    path = Path(path)
    obj = read_json_object(path)
    arch = get_architecture(architecture_name_of(obj, str(path)))
    return arch, arch.read_config(obj, str(path))
