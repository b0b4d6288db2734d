"""The parts models are put together from, and their registries."""
from .base import (  # noqa: F401
    PagedKV,
    Part,
    Runtime,
    SlotState,
    TensorSpec,
    build_part,
    register_part,
)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401,E402
from .model import Model, expected_tensors  # noqa: F401,E402
