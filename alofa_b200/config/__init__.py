"""Typed configuration: the strict JSON reader, the architecture registry, the
architecture-neutral model description and the engine's own settings."""
from .engine_config import EngineConfig  # noqa: F401
from .json_reader import Keys, read_json_object  # noqa: F401
from .registry import (  # noqa: F401
    Architecture,
    get_architecture,
    known_architectures,
    read_model_config,
    register_architecture,
)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry  # noqa: F401
