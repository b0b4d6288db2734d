"""Random weights from a configuration and a seed.

Matrices and biases are drawn from N(0, 0.02), norm weights from
1 + N(0, 0.01).  Every tensor has its own generator, seeded from the seed and
the tensor's name, so a tensor's values do not depend on which other tensors
exist or in which order they are made.  The reference has no such mode (its
tests use the real checkpoint or no model at all)."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..config.registry import get_architecture
from ..errors import AlofaError
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(seed: int, name: str, shape, init: str, dtype, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    x = torch.randn(tuple(shape), generator=gen, dtype=torch.float32, device=device)
    if init == "normal":
        x.mul_(0.02)
    elif init == "ones":
        x.mul_(0.01).add_(1.0)
    else:
        raise AlofaError("invalid_argument", "unknown init law", f"name={name} init={init}")
    return x.to(dtype)


def random_state(model_tensors: dict, seed: int, dtype=torch.bfloat16, device="cpu") -> dict:
    """``model_tensors``: name -> TensorSpec (see parts.base).  Optional
    tensors are not made."""
    out = {}
    for name, spec in model_tensors.items():
        if spec.optional:
            continue
        out[name] = random_tensor(seed, name, spec.shape, spec.init, dtype, device)
    return out


def write_random_model(folder, architecture: str, config, seed: int, dtype=torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a typed config."""
    from ..parts.model import expected_tensors

    arch = get_architecture(architecture)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    spec = arch.build_spec(config)
    tensors = random_state(expected_tensors(spec), seed, dtype)
    (folder / "config.json").write_text(json.dumps(arch.to_json(config), indent=1) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": seed})
    return folder
