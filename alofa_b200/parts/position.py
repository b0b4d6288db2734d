"""Position encodings.

``rotary_neox`` is the half-split rotary encoding: for position p and pair
index i < rot/2, ``inv_i = f32(1) / f32(theta^(2i/rot))`` with the power in
f64, ``angle = f32(p) * inv_i`` as an fp32 product, and cos/sin taken in f64
and rounded once to fp32 (src/alofa/model/arch/qwen.mojo:830-880).  The
rotation itself, ``y[d] = a cos - b sin``, ``y[d + rot/2] = b cos + a sin``
(src/alofa/kernels/cpu/scalar.mojo:283-344), runs inside the mixer's
rotate-and-store kernel, which reads the table built here."""
from __future__ import annotations

import numpy as np
import torch

from ..errors import AlofaError
from .base import Part, register_part


class RotaryNeox(Part):
    family = "position"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.head_dim = int(self.param("head_dim"))
        self.rotary_dim = int(self.param("rotary_dim", self.head_dim))
        self.theta = float(self.param("theta"))
        self.max_position = int(self.param("max_position"))
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise AlofaError("unsupported", "rotary_dim must be even, positive and at most head_dim", f"rotary_dim={self.rotary_dim} head_dim={self.head_dim}")
        self._table = None

    def key(self):
        return ("rotary_neox", self.rotary_dim, self.theta, self.max_position)

    def build_table(self, n_positions: int) -> torch.Tensor:
        """[n_positions, rot/2, 2] fp32 (cos, sin) on the device."""
        half = self.rotary_dim // 2
        i = np.arange(half, dtype=np.float64)
        inv = np.float32(1.0) / np.power(np.float64(self.theta), 2.0 * i / self.rotary_dim).astype(np.float32)
        pos = np.arange(n_positions, dtype=np.float32)
        angle = (pos[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)
        table = np.stack([np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)], axis=-1)
        return torch.from_numpy(np.ascontiguousarray(table)).to(self.rt.device)

    def load(self, state):
        # one table per distinct (rot, theta, length) is shared through the state dict
        tables = state.setdefault("__rotary_tables__", {})
        if self.key() not in tables:
            tables[self.key()] = self.build_table(self.max_position)
        self._table = tables[self.key()]

    def rotary_table(self):
        """(table, rotary_dim) for the fused rotate-and-store kernel."""
        return self._table, self.rotary_dim


class NoPosition(Part):
    """No position encoding: queries and keys are used as projected."""

    family = "position"
    graph_safe = True

    def rotary_table(self):
        return None, 0


register_part("position", "rotary_neox", RotaryNeox)
register_part("position", "none", NoPosition)
