"""Matrix products of the parts: ``y = x W^T (+ b)`` with the epilogue fused.

One :class:`Linear` holds a weight ``[out, in]`` (row-major, as stored in the
checkpoint; src/alofa/kernels/cpu/scalar.mojo:10-18) and picks the kernel per
call: the tensor-core kernel when the operands are bfloat16 and the sizes are
ones it takes, else the generic FMA kernel, which takes every size and is the
only one the 32-bit path uses.

When the tensor-core kernel splits the depth over several CTAs it leaves
partial sums; a caller whose next kernel can add them up while reading (the
norm that follows a residual product, the rotate-and-store that follows q/k/v)
asks for them with ``defer=True`` and gets a :class:`Partial` back instead of a
finished output."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..csrc import ops
from ..errors import AlofaError

STORE, RESIDUAL, GATED = ops.EPI_STORE, ops.EPI_RESIDUAL, ops.EPI_GATED


@dataclass
class Partial:
    """Split-K partial sums ``[splits, tokens, features]`` (fp32) that still
    have to be added up, with the bias that goes on top."""

    sums: torch.Tensor
    splits: int
    bias: Optional[torch.Tensor]


class MergedSplits:
    """Rows a product may read that are not in memory yet: the attention
    output of decode tokens, still split by keys (``partial_o [splits, T *
    heads, head_dim]``, ``partial_ml [splits, T * heads, 2]``).  A product that
    can merges them while it loads its operand; any other consumer calls
    :meth:`rows`."""

    dtype = torch.bfloat16

    def __init__(self, partial_o, partial_ml, positions, tokens: int, heads: int, head_dim: int, window, split_keys: int, buf):
        self.partial_o, self.partial_ml, self.positions = partial_o, partial_ml, positions
        self.buf = buf  # the step's scratch allocator
        self.heads, self.head_dim, self.window, self.split_keys = heads, head_dim, window, split_keys
        self.shape = (tokens, heads * head_dim)

    def fits_kernel(self) -> bool:
        return self.partial_o.shape[0] <= 16

    def computed(self):
        return (ops.B_MERGED_SPLITS, self.partial_o, self.partial_ml, self.positions, self.heads, self.head_dim, self.window, self.split_keys)

    def rows(self) -> torch.Tensor:
        out = self.buf(self.shape, torch.bfloat16)
        ops.attention_combine(out, self.partial_o, self.partial_ml, self.positions, self.heads, self.head_dim, self.window, self.split_keys)
        return out


class NormedRows:
    """Rows a product may read that are not in memory yet: the RMSNorm of the
    residual stream ``h``, which a decode step of a few tokens keeps as a base
    tensor plus a fixed-point accumulator.  A product that can makes the rows
    while it loads its operand (:meth:`computed`, then :meth:`done`); any other
    consumer calls :meth:`rows`, which runs the norm kernel."""

    dtype = torch.bfloat16
    kind = "normed"

    def __init__(self, ctx, h, norm):
        self.ctx, self.h, self.norm = ctx, h, norm
        self.shape = (h.shape[0], norm.size)
        self._pend = None

    def fits_kernel(self) -> bool:
        pend = self.ctx.pending
        return pend is None or pend.h is not self.h or pend.partial is None  # planes are added by the norm kernel, not here

    def computed(self):
        """``(B_NORMED, base, acc or None, gamma, eps, new_base, zero or
        None)``; the stream's duty passes to the product that takes this."""
        ctx, h = self.ctx, self.h
        pend = self._pend = ctx.take_pending(h)
        base = pend.base if pend is not None else h
        acc = zero = None
        if pend is not None and pend.acc is not None:
            st = ctx.stream_of(h)
            acc, zero = st["acc"][pend.acc], st["acc"][1 - pend.acc]
        return (ops.B_NORMED, base, acc, self.norm.weight, self.norm.eps, ctx.other_base(h, base), zero)

    def done(self, computed) -> None:
        """The product ran: the stream's base is now ``computed``'s new base."""
        self.ctx.stream_read(self.h, computed[5], self._pend)

    def undo(self) -> None:
        """The product refused after all: the stream is as it was."""
        self.ctx.pending = self._pend

    def rows(self) -> torch.Tensor:
        return self.norm.rows_now(self.ctx, self.h)


ACCUMULATED = object()  # what a residual product returns when it added its sums into the stream's accumulator


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

    def can_accumulate(self, tokens: int) -> bool:
        """Whether a call with this many tokens can add its sums into a stream
        accumulator (``acc``): the tensor-core kernel with the weights on the
        M side, a residual product."""
        return self._fast is not None and self.epi == RESIDUAL and self._fast.weights_on_m(tokens)

    def __call__(self, out: Optional[torch.Tensor], x, defer: bool = False, buf=None, acc=None):
        """Run the product.  ``x`` is a tensor of rows, or rows still to be
        made (:class:`MergedSplits`, :class:`NormedRows`).  With ``defer`` the
        result may come back as a :class:`Partial` (``out`` is then
        untouched); else None.  ``buf(shape, dtype)`` is the step's scratch
        allocator (``ctx.buf``), used for split sums; without it they are
        allocated.  ``acc`` (only after :meth:`can_accumulate`): the sums are
        added into this int64 accumulator instead of into ``out``, and
        ``ACCUMULATED`` is returned."""
        if acc is not None:
            if x.dtype != torch.bfloat16 or self._fast(out, x, False, buf, acc) is not ACCUMULATED:
                raise AlofaError("state", "a product that was to add into the stream's accumulator could not")
            return ACCUMULATED
        if self._fast is not None and x.dtype == torch.bfloat16:
            done = self._fast(out, x, defer, buf)
            if done is not False:
                return done if isinstance(done, Partial) else None
        if not isinstance(x, torch.Tensor):
            x = x.rows()
        ops.gemm_generic(out, x, self.weight, self.bias, self.epi)
        return None


def add_into_stream(ctx, linear: Linear, h, x) -> None:
    """``h += linear(x)`` for a product into the residual stream: into the
    stream's accumulator where the step keeps one, else as split sums left for
    the next reader of ``h`` to add, else in place."""
    acc = ctx.accumulator_for(h) if linear.can_accumulate(x.shape[0]) else None
    if acc is not None:
        linear(h, x, buf=ctx.buf, acc=acc)
        ctx.owe_accumulator(h)
        return
    if ctx.pending is not None and ctx.pending.h is h and (ctx.pending.acc is not None or ctx.pending.base is not h):
        ctx.flush_pending()  # the product adds in place or leaves planes on top of h itself
    owed = linear(h, x, defer=True, buf=ctx.buf)
    if owed is not None:
        ctx.set_pending(h, owed)
