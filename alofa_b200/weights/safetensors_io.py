"""Reading and writing single-file safetensors.

Layout: an 8-byte little-endian header length, a JSON header mapping each
tensor name to ``dtype``, ``shape`` and ``data_offsets`` (relative to the end
of the header), then the raw little-endian data.  The checks are the
reference's (src/alofa/model/safetensors.mojo:147-303): header inside the
file, ``__metadata__`` skipped, byte range equal to shape times element size,
range inside the file, empty header refused; F16 is parsed but refused by
name when used, other dtypes are refused at parse."""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch

from ..errors import AlofaError

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass
class TensorEntry:
    name: str
    dtype: str
    shape: tuple
    begin: int  # absolute file offsets
    end: int


class SafeTensorFile:
    """A memory-mapped safetensors file; tensors are views of the mapping
    until they are copied to the device."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as err:
            raise AlofaError("io", "cannot open weight file", f"file={self.path}: {err}") from err
        size = self.path.stat().st_size
        if size < 8:
            raise AlofaError("parse", "weight file is shorter than its header length", f"file={self.path} size={size}")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen == 0 or 8 + hlen > size:
            raise AlofaError("parse", "safetensors header length is outside the file", f"file={self.path} header={hlen} size={size}")
        try:
            header = json.loads(self._map[8 : 8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as err:
            raise AlofaError("parse", "safetensors header is not valid JSON", f"file={self.path}: {err}") from err
        base = 8 + hlen
        self.entries = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dtype = meta.get("dtype")
            if dtype not in _DTYPES:
                raise AlofaError("unsupported", "tensor dtype is not supported", f"name={name} dtype={dtype} file={self.path}")
            shape = tuple(int(d) for d in meta["shape"])
            lo, hi = (int(x) for x in meta["data_offsets"])
            count = 1
            for d in shape:
                count *= d
            if hi - lo != count * _DTYPES[dtype][1]:
                raise AlofaError("parse", "tensor byte range does not match its shape", f"name={name} shape={shape} bytes={hi - lo} file={self.path}")
            if lo < 0 or base + hi > size:
                raise AlofaError("parse", "tensor byte range is outside the file", f"name={name} file={self.path}")
            self.entries[name] = TensorEntry(name, dtype, shape, base + lo, base + hi)
        if not self.entries:
            raise AlofaError("parse", "safetensors file holds no tensor", f"file={self.path}")

    def names(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only; copy before writing)."""
        if name not in self.entries:
            raise AlofaError("invalid_argument", "entry is not in the file", f"name={name} file={self.path}")
        e = self.entries[name]
        if e.dtype == "F16":
            raise AlofaError("unsupported", "float16 tensors are not supported", f"name={name} file={self.path}")
        dtype, width = _DTYPES[e.dtype]
        count = (e.end - e.begin) // width
        if count == 0:
            return torch.empty(e.shape, dtype=dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the mapping is read-only; nothing writes through the view
            flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=e.begin)
        return flat.view(e.shape)

    def close(self):
        try:
            self._map.close()
        except BufferError:
            pass  # views are still alive; the mapping goes with them
        self._fh.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names, data 16-byte aligned per tensor in
    the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise AlofaError("unsupported", "cannot write this dtype", f"name={name} dtype={t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        blobs.append(t)
        offset += nbytes
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((-(8 + len(text))) % 16)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for t in blobs:
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
