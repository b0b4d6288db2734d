"""Sampling: settings, the per-request bit source, and the device kernels' face."""
from .params import SamplingParams  # noqa: F401
from .rng import SplitMix64  # noqa: F401
