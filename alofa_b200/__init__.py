"""alofa_b200: a single-GPU inference engine for decoder language models on
NVIDIA B200 (sm_100a), built around paged caches, one batched step function and
hand-written CUDA kernels.

Public entry points:

* :class:`alofa_b200.engine.Engine` - load a model folder and generate tokens.
* ``python -m alofa_b200.cli.generate`` - the command line of the same.
* ``bin/trace_run`` - feed given token ids step by step and dump logits.
"""

__version__ = "0.1.0"

from .errors import AlofaError  # noqa: F401
