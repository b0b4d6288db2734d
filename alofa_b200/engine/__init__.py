"""The engine: step function, scheduler, generation loop."""
from .step import StepEntry, StepRunner  # noqa: F401


def __getattr__(name):
    if name in ("Engine", "SamplingParams", "load_model"):
        from . import engine

        return getattr(engine, name)
    raise AttributeError(name)
