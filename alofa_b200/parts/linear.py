"""Matrix products of the parts: ``y = x W^T (+ b)`` with the epilogue fused.

One :class:`Linear` holds a weight ``[out, in]`` (row-major, as stored in the
checkpoint; src/alofa/kernels/cpu/scalar.mojo:10-18) and picks the kernel per
call: the tensor-core kernel when the operands are bfloat16 and the sizes are
ones it takes, else the generic FMA kernel, which takes every size and is the
only one the 32-bit path uses."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError

STORE, RESIDUAL, GATED = ops.EPI_STORE, ops.EPI_RESIDUAL, ops.EPI_GATED


class Linear:
    """``epi`` STORE: out = x W^T + b.  RESIDUAL: out (fp32) += x W^T + b.
    GATED: W = [gate; up]: out = silu(x Wg^T) * (x Wu^T)."""

    def __init__(self, weight: torch.Tensor, bias, epi: int = STORE):
        self.weight = weight.contiguous()
        self.bias = bias
        self.epi = epi
        rows, self.in_features = self.weight.shape
        if epi == GATED and rows % 2:
            raise AlofaError("invalid_argument", "a gated weight needs an even number of rows", f"rows={rows}")
        self.out_features = rows // 2 if epi == GATED else rows
        self._fast = None
        if self.weight.dtype == torch.bfloat16:
            from . import fast_linear

            self._fast = fast_linear.plan(self)

    def __call__(self, out: torch.Tensor, x: torch.Tensor) -> None:
        if self._fast is not None and x.dtype == torch.bfloat16 and self._fast(out, x):
            return
        ops.gemm_generic(out, x, self.weight, self.bias, self.epi)
