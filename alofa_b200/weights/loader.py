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
src/alofa/model/safetensors.mojo:123-137).  Integer tables become int32.

A folder holds either ``model.safetensors`` or, as the large published
checkpoints do, several shard files with ``model.safetensors.index.json``
whose ``weight_map`` names the shard of every tensor (the reference reads the
single file only, src/alofa/model/loader.mojo:106-224).  All shards are
opened first and compared with the model at once, so the one error also covers
a tensor that the index places in a shard that does not hold it, and a tensor
that two shards hold.

To the device: the files are memory-mapped; each tensor goes through two
pinned staging buffers in turn (the copy of one chunk to the device runs while
the next chunk is read from the mapping) into device memory of its own."""
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


STAGE_BYTES = 64 << 20


class _Staging:
    """Two pinned buffers used in turn for host-to-device copies."""

    def __init__(self, device):
        self.device = device
        self.buffers = [torch.empty(STAGE_BYTES, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.events = [None, None]
        self.turn = 0

    def to_device(self, t: torch.Tensor) -> torch.Tensor:
        """A device copy of the CPU tensor ``t`` (a view of a mapped file)."""
        src = t.contiguous().view(-1).view(torch.uint8)
        out = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        dst = out.view(-1).view(torch.uint8)
        for lo in range(0, src.numel(), STAGE_BYTES):
            hi = min(lo + STAGE_BYTES, src.numel())
            i = self.turn
            self.turn ^= 1
            if self.events[i] is not None:
                self.events[i].synchronize()  # the copy that last used this buffer is done
            self.buffers[i][: hi - lo].copy_(src[lo:hi])
            dst[lo:hi].copy_(self.buffers[i][: hi - lo], non_blocking=True)
            self.events[i] = torch.cuda.Event()
            self.events[i].record()
        return out

    def finish(self) -> None:
        for ev in self.events:
            if ev is not None:
                ev.synchronize()


INDEX_NAME = "model.safetensors.index.json"


def open_checkpoint(folder) -> tuple:
    """([opened files], name -> file, problems) of a model folder: the single
    ``model.safetensors``, or the shards its index names."""
    folder = Path(folder)
    single, index = folder / "model.safetensors", folder / INDEX_NAME
    if not index.exists():
        if not single.exists():
            raise AlofaError("io", "model folder has no model.safetensors and no " + INDEX_NAME, f"folder={folder}")
        st = SafeTensorFile(single)
        return [st], {n: st for n in st.names()}, []
    from ..config.json_reader import read_json_object

    weight_map = read_json_object(index).get("weight_map")
    if not isinstance(weight_map, dict) or not weight_map:
        raise AlofaError("parse", "the shard index has no weight_map", f"file={index}")
    files, where, problems = {}, {}, []
    try:
        for shard in sorted(set(weight_map.values())):
            if not isinstance(shard, str) or "/" in shard or "\\" in shard:
                raise AlofaError("parse", "the shard index names a file outside the model folder", f"file={index} shard={shard}")
            if not (folder / shard).exists():
                raise AlofaError("io", "a shard named by the index is missing", f"folder={folder} shard={shard}")
            files[shard] = SafeTensorFile(folder / shard)
        holders = {}
        for shard, st in files.items():
            for n in st.names():
                holders.setdefault(n, []).append(shard)
        for n, shards in sorted(holders.items()):
            if len(shards) > 1:
                problems.append(f"{n} is held by {len(shards)} shards: {', '.join(shards)}")
        for n, shard in sorted(weight_map.items()):
            if n in files[shard].entries:
                where[n] = files[shard]
            else:
                problems.append(f"{n} is not in {shard}, where the index places it")
        for n, shards in sorted(holders.items()):
            if n not in weight_map:
                where.setdefault(n, files[shards[0]])  # reported as unexpected unless the model wants it
    except Exception:
        for st in files.values():
            st.close()
        raise
    return list(files.values()), where, problems


def load_state(expected: dict, source, compute_dtype: torch.dtype, device) -> dict:
    """name -> device tensor.  ``source`` is a model folder or a dict of
    CPU/GPU tensors (the in-memory random mode)."""
    if isinstance(source, dict):
        found = {n: tuple(t.shape) for n, t in source.items()}
        check_names_and_shapes(expected, found, "in-memory state")
        return {n: _place(t, compute_dtype, device) for n, t in source.items()}
    files, where, problems = open_checkpoint(source)
    try:
        found = {n: st.entries[n].shape for n, st in where.items()}
        try:
            check_names_and_shapes(expected, found, str(source))
        except AlofaError as err:
            if problems:
                raise AlofaError(err.code, err.message, err.detail + " | shard index (" + str(len(problems)) + "): " + "; ".join(problems)) from None
            raise
        if problems:
            raise AlofaError("invalid_argument", "weights do not match the model", f"shard index ({len(problems)}): " + "; ".join(problems) + f" | source={source}")
        on_gpu = torch.device(device).type == "cuda"
        staging = _Staging(device) if on_gpu else None
        out = {}
        for n, st in where.items():
            t = st.tensor(n)
            if on_gpu:
                out[n] = _place(staging.to_device(t), compute_dtype, device)
            else:
                out[n] = _place(t, compute_dtype, device).clone()
        if staging is not None:
            staging.finish()
        return out
    finally:
        for st in files:
            st.close()
