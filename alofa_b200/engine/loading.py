"""From a model folder (or a configuration and a seed) to a loaded model.

The reference does the same in ``QwenModel`` construction: config.json read
into ``QwenConfig`` (src/alofa/model/arch/qwen.mojo:929-982), tensors bound by
their Hugging Face names with the required-name list checked at once
(qwen.mojo:1168-1189)."""
from __future__ import annotations

import torch

from ..config.registry import get_architecture, read_model_config
from ..errors import AlofaError
from ..parts.base import Runtime
from ..parts.model import Model
from ..weights.loader import load_state
from ..weights.random_init import random_state

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def compute_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        name = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(name, str(name))
    if name not in _DTYPES:
        raise AlofaError("invalid_argument", "dtype must be bfloat16 or float32", f"dtype={name}")
    return _DTYPES[name]


def require_cuda(device=None) -> torch.device:
    """The engine runs on a CUDA device only; there is no CPU path."""
    if not torch.cuda.is_available():
        raise AlofaError("unsupported", "alofa_b200 needs a CUDA device (sm_100a); none is visible")
    dev = torch.device(device or "cuda:0")
    if dev.type != "cuda":
        raise AlofaError("unsupported", "alofa_b200 runs on CUDA devices only", f"device={dev}")
    return dev


def load_model(folder, dtype="bfloat16", device=None):
    """(model, typed config, architecture) of a folder with config.json and
    model.safetensors; the model class is chosen by config.json."""
    dev = require_cuda(device)
    arch, cfg = read_model_config(folder)
    spec = arch.build_spec(cfg)
    model = Model(spec, Runtime(dev, compute_dtype(dtype)))
    state = load_state(model.tensors(), folder, model.rt.dtype, dev)
    model.load(state)
    return model, cfg, arch


def random_model(architecture: str, config, seed: int, dtype="bfloat16", device=None, generate_on_device: bool = False):
    """A model with seeded random weights, without a folder on disk.  With
    ``generate_on_device`` the numbers are drawn by the device's generator
    (fast for large shapes; a different stream than the CPU's)."""
    dev = require_cuda(device)
    arch = get_architecture(architecture)
    spec = arch.build_spec(config)
    model = Model(spec, Runtime(dev, compute_dtype(dtype)))
    state = random_state(model.tensors(), seed, torch.bfloat16, dev if generate_on_device else "cpu")
    model.load(load_state(model.tensors(), state, model.rt.dtype, dev))
    return model, config, arch
