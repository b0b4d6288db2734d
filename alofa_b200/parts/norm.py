"""RMSNorm: ``y = x / sqrt(mean(x^2) + eps) * w`` per row, fp32 sums; no bias,
no mean subtraction, the weight is used as stored
(src/alofa/kernels/cpu/scalar.mojo:93-129)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, TensorSpec, as_float32_vector, register_part
from .linear import NormedRows


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
    gives_normed_rows = True  # forward(lazy=True) may hand its reader rows still to be made

    def scratch_row_bytes(self) -> int:
        return 4 * self.size

    def forward(self, ctx, h, rows=None, lazy=False):
        """Normalised rows of the fp32 stream ``h`` in the compute dtype;
        ``rows`` (int32 on the device) picks rows of ``h``.  With ``lazy`` the
        caller's next product can make normalised rows itself from the stream:
        it then gets a :class:`~alofa_b200.parts.linear.NormedRows` (nothing is
        launched) where the step keeps the stream as base + accumulator."""
        if lazy and rows is None and ctx.stream_of(h) is not None and h.shape[1] == self.size:
            return NormedRows(ctx, h, self)
        return self.rows_now(ctx, h, rows)

    def rows_now(self, ctx, h, rows=None):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = ctx.buf((n, self.size), self.rt.dtype)
        pend = ctx.take_pending(h)
        if pend is not None and pend.acc is not None:
            acc, other = ctx.accumulators(h, pend)
            if rows is None and ops.norm_fused(out, h, self.weight, self.eps, None, base=pend.base if pend.base is not h else None, acc=acc, other=other):
                return out
            ops.stream_settle(h, pend.base, acc, other)  # picked rows, or a width the fused kernel refuses: the whole stream first
            pend = None
        if pend is not None and pend.partial is None and pend.base is not h:
            h.copy_(pend.base)
            pend = None
        if pend is not None:
            owed = pend.partial
            base = pend.base if pend.base is not h else None
            if rows is None or base is None:
                if ops.norm_fused(out, h, self.weight, self.eps, rows, owed.sums, owed.splits, owed.bias, base=base if rows is None else None):
                    return out
            if base is not None:
                h.copy_(base)
            ops.splitk_reduce(h, owed.sums, owed.bias, owed.splits, ops.EPI_RESIDUAL)
        if self.rt.dtype == torch.bfloat16 and ops.norm_fused(out, h, self.weight, self.eps, rows):
            return out
        ops.rmsnorm(out, h, self.weight, self.eps, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
