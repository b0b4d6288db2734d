"""RMSNorm: ``y = x / sqrt(mean(x^2) + eps) * w`` per row, fp32 sums; no bias,
no mean subtraction, the weight is used as stored
(src/alofa/kernels/cpu/scalar.mojo:93-129)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, TensorSpec, as_float32_vector, register_part


class RMSNorm(Part):
    family = "norm"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))
        self.weight = None

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.size,), "ones")}

    def load(self, state):
        self.weight = as_float32_vector(state[self.prefix + "weight"])

    absorbs_pending = True  # adds split-K partial sums owed to h while reading it

    def scratch_row_bytes(self) -> int:
        return 4 * self.size

    def forward(self, ctx, h, rows=None):
        """Normalised rows of the fp32 stream ``h`` in the compute dtype;
        ``rows`` (int32 on the device) picks rows of ``h``."""
        n = h.shape[0] if rows is None else rows.shape[0]
        out = ctx.buf((n, self.size), self.rt.dtype)
        owed = ctx.take_pending(h)
        if owed is not None:
            if ops.norm_fused(out, h, self.weight, self.eps, rows, owed.sums, owed.splits, owed.bias):
                return out
            ops.splitk_reduce(h, owed.sums, owed.bias, owed.splits, ops.EPI_RESIDUAL)
        if self.rt.dtype == torch.bfloat16 and ops.norm_fused(out, h, self.weight, self.eps, rows):
            return out
        ops.rmsnorm(out, h, self.weight, self.eps, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
