"""Weights: the safetensors reader and writer, the checked loader and the
seeded random-weights mode."""
from .loader import check_names_and_shapes, load_state  # noqa: F401
from .random_init import random_state, write_random_model  # noqa: F401
from .safetensors_io import SafeTensorFile, write_safetensors  # noqa: F401
