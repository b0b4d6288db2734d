"""Weights by tensor name, checked against what the model expects.

The model's parts say which tensors they need (name, shape); the loader
compares that list with the file once and raises ONE error that lists every
missing tensor, every unexpected tensor and every wrong shape, instead of
failing on the first (the reference checks names one by one at construction,
src/alofa/model/arch/qwen.mojo:1168-1189, and names a missing entry,
src/alofa/model/loader.mojo:235-248).

Dtypes: a tensor stored as BF16 stays bfloat16 and a tensor stored as F32
stays float32 when the engine runs in bfloat16; when it runs in float32
everything is widened to float32 (bf16 widening is exact,
src/alofa/model/safetensors.mojo:123-137).  Integer tables become int32."""
from __future__ import annotations

from pathlib import Path

import torch

from ..errors import AlofaError
from .safetensors_io import SafeTensorFile


def check_names_and_shapes(expected: dict, found: dict, origin: str) -> None:
    """``expected``: name -> TensorSpec; ``found``: name -> shape tuple."""
    missing = [n for n, s in expected.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in expected]
    wrong = [
        f"{n} got={tuple(found[n])} want={tuple(s.shape)}"
        for n, s in expected.items()
        if n in found and tuple(found[n]) != tuple(s.shape)
    ]
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append(f"wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise AlofaError("invalid_argument", "weights do not match the model", " | ".join(parts) + f" | source={origin}")


def _place(t: torch.Tensor, compute_dtype: torch.dtype, device) -> torch.Tensor:
    if t.dtype in (torch.int64, torch.int32):
        return t.to(device=device, dtype=torch.int32)
    if compute_dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32)
    return t.to(device=device)  # stored dtype kept: bf16 stays bf16, f32 stays f32


def load_state(expected: dict, source, compute_dtype: torch.dtype, device) -> dict:
    """name -> device tensor.  ``source`` is a model folder (model.safetensors
    inside it) or a dict of CPU/GPU tensors (the in-memory random mode)."""
    if isinstance(source, dict):
        found = {n: tuple(t.shape) for n, t in source.items()}
        check_names_and_shapes(expected, found, "in-memory state")
        return {n: _place(t, compute_dtype, device) for n, t in source.items()}
    path = Path(source) / "model.safetensors"
    if not path.exists():
        raise AlofaError("io", "model folder has no model.safetensors", f"folder={source}")
    st = SafeTensorFile(path)
    try:
        found = {n: e.shape for n, e in st.entries.items()}
        check_names_and_shapes(expected, found, str(path))
        return {n: _place(st.tensor(n), compute_dtype, device).clone() if device == "cpu" else _place(st.tensor(n), compute_dtype, device) for n in st.names()}
    finally:
        st.close()
