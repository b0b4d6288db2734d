"""A decode step as a program for one resident kernel.

With a few tokens per step the kernels of a layer take a microsecond or two
each and the step's time goes to the gaps between them.  A
:class:`DecodeProgram` is the same step as data: a list of phases (embedding,
products with fused epilogues, attention over the cache, the merge of its
splits) that one cooperative kernel works through, a barrier over the grid
between two phases (``csrc/kernels/decode_program.cu``).

The parts of a model write the list: a part that can run inside a program has
an ``emit`` method beside ``forward``, which calls the methods below instead
of launching kernels.  ``emit`` of a norm returns an :class:`Operand` that
stands for "these rows, normalised"; the product that consumes it normalises
on the way in.  A part without ``emit``, or a size the kernel does not take,
raises :class:`Ineligible`, and the step is launched kernel by kernel as
before.  The counterpart in the reference is the per-layer call sequence of
``BatchExecutor.forward`` (src/alofa/engine/executor.mojo:745-859)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from ..csrc import ops
from ..parts.base import Ineligible


@dataclass
class Operand:
    """Rows that a product reads: bfloat16 rows as they are, or rows of the
    fp32 stream to be normalised (``gamma``, ``eps``) on the way in."""

    rows: torch.Tensor
    gamma: Optional[torch.Tensor] = None
    eps: float = 0.0


class DecodeProgram:
    # epilogues of a product
    STORE_BF16, STORE_F32, RESIDUAL, GATED, ROPE_STORE = 0, 1, 2, 3, 4

    def __init__(self, ctx):
        if ctx.rt.dtype != torch.bfloat16 or ctx.n_tokens != ctx.n_seqs or ctx.n_tokens > ops.PROGRAM_MAX_TOKENS:
            raise Ineligible("a program runs bfloat16 steps of at most 16 requests with one token each")
        self.ctx = ctx
        self.n = ctx.n_tokens
        self.head_dim = None
        self._phases = []      # filled descriptors (bytes)
        self._keep = []        # tensors the descriptors point to
        self._device = None
        self._smem = 0
        self._sync = None
        self.logits = None

    # -- what parts call ------------------------------------------------------
    def buf(self, shape, dtype) -> torch.Tensor:
        """Scratch that lives as long as the program."""
        t = torch.empty(shape, dtype=dtype, device=self.ctx.rt.device)
        self._keep.append(t)
        return t

    def normed(self, h: torch.Tensor, gamma: torch.Tensor, eps: float) -> Operand:
        if h.dtype != torch.float32 or gamma.dtype != torch.float32:
            raise Ineligible("a normalised operand reads the fp32 stream")
        return Operand(h, gamma, float(eps))

    def rows(self, x: torch.Tensor) -> Operand:
        if x.dtype != torch.bfloat16:
            raise Ineligible("a plain operand is bfloat16")
        return Operand(x)

    def embed(self, h, table, ids, src=None, fed=None) -> None:
        """h[t] = table[ids[t]], or table[fed[src[t]]] where src[t] >= 0."""
        if table.dtype != torch.bfloat16:
            raise Ineligible("the embedding table is not bfloat16")
        self._keep += [h, table, ids, src, fed]
        ptr = lambda t: t.data_ptr() if t is not None else None
        self._add(lambda lib, ph: lib.alofa_program_embed(ph, h.data_ptr(), table.data_ptr(), ids.data_ptr(), ptr(src), ptr(fed), self.n, table.shape[1], table.shape[0]))

    def linear(self, x: Operand, weight, bias, epi: int, out: torch.Tensor) -> None:
        """out = x W^T (+ bias) with epilogue ``epi`` (STORE_BF16, STORE_F32,
        RESIDUAL: out += ..., GATED: W = [gate; up], out = silu(gate) * up)."""
        self._linear(x, weight, bias, epi, out, out.shape[1])

    def rope_store(self, x: Operand, weight, bias, q, k_cache, v_cache, slot_map, positions, table, nh, nkv, hd, writes: bool) -> None:
        """W = [q; k; v] stacked (q only when the layer reads another's cache):
        bias, rotation of q and k by the cos/sin table, q to ``q``, k and v to
        their cache slots."""
        self._head_dim(hd)
        self._keep += [q, k_cache, v_cache, slot_map, positions, table]
        self._linear(x, weight, bias, self.ROPE_STORE, None, 0, (q, k_cache, v_cache, slot_map, positions, table, nh, nkv, writes))

    def attention(self, out, q, k_cache, v_cache, kv_len, block_table, page_size, nh, nkv, hd, window, scale, max_context) -> None:
        """out = attention of each request's one token over its cached keys."""
        self._head_dim(hd)
        lib = self._lib()
        splits = lib.alofa_program_splits(int(max_context))
        po = self.buf((splits, self.n * nh, hd), torch.float32)
        pml = self.buf((splits, self.n * nh, 2), torch.float32)
        counters = torch.zeros(self.n * nkv, dtype=torch.int32, device=self.ctx.rt.device)
        self._keep += [out, q, k_cache, v_cache, kv_len, block_table, counters]
        self._add(lambda lib, ph: lib.alofa_program_attention(
            ph, out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0], kv_len.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], page_size, self.n, nh, nkv, int(window or 0), float(scale), int(max_context), po.data_ptr(), pml.data_ptr(),
            counters.data_ptr()))

    # -- building and running ---------------------------------------------------
    def _head_dim(self, hd: int) -> None:
        if not ops.program_supported(hd) or self.head_dim not in (None, hd):
            raise Ineligible(f"head size {hd} (one of 64 and 128 for the whole program)")
        self.head_dim = hd

    def _lib(self):
        return ops.program_library(self.head_dim or 64)

    def _add(self, fill) -> None:
        self._phases.append(fill)

    def _linear(self, x, weight, bias, epi, out, out_cols, rope=None) -> None:
        if weight.dtype != torch.bfloat16 or not weight.is_contiguous() or weight.shape[1] != x.rows.shape[1]:
            raise Ineligible("a product's weight is bfloat16 [out, in], rows contiguous")
        if bias is not None and bias.dtype != torch.float32:
            raise Ineligible("a bias is fp32")
        self._keep += [x.rows, weight, bias, out, x.gamma]
        n_rows, depth = weight.shape
        grid = ops.program_grid()
        q, kc, vc, slot_map, positions, table, nh, nkv, writes = rope or (None,) * 6 + (0, 0, 0)
        ptr = lambda t: t.data_ptr() if t is not None else None
        self._add(lambda lib, ph: lib.alofa_program_linear(
            ph, 1 if x.gamma is not None else 0, x.rows.data_ptr(), ptr(x.gamma), x.eps, weight.data_ptr(), ptr(bias), ptr(out), epi,
            self.n, n_rows, depth, out_cols, 0, ptr(q), ptr(kc), ptr(vc), ptr(slot_map), ptr(positions), ptr(table), nh, nkv, int(bool(writes)), grid))

    def finish(self) -> None:
        """Fill the descriptors and copy them to the device."""
        lib = self._lib()
        size = lib.alofa_program_phase_bytes()
        host = ctypes.create_string_buffer(size * len(self._phases))
        base = ctypes.addressof(host)
        for i, fill in enumerate(self._phases):
            if fill(lib, base + i * size) != 0:
                raise Ineligible(f"phase {i} has a size the program kernel does not take")
        self._smem = lib.alofa_program_smem_bytes(base, len(self._phases))
        if self._smem > ops.PROGRAM_MAX_SMEM:
            raise Ineligible("the operands of a product do not fit in shared memory")
        self._device = torch.frombuffer(bytearray(host.raw), dtype=torch.uint8).to(self.ctx.rt.device)
        self._sync = torch.zeros(1, dtype=torch.int32, device=self.ctx.rt.device)
        self.n_phases = len(self._phases)
        self._phases = None

    def run(self) -> None:
        ops.program_run(self._lib(), self._device, self.n_phases, self._sync, self.ctx.status, self._smem)
