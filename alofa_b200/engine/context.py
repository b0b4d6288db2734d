"""What one step tells the parts about its batch.

A step runs ``n_tokens`` packed rows belonging to ``n_seqs`` requests; each
request contributes one contiguous run of rows (a portion of its prompt, or
one decoded token).  Everything the kernels index with lives in ONE int32
device buffer filled by one host-to-device copy; the fields below are views
into it.  The layout depends only on (tokens, requests, wanted rows), so a
captured CUDA graph of a given shape sees the same addresses every replay.
The reference's counterpart is the per-row metadata its executor plans
(``row_tok, row_pos, row_req, out_rows``: src/alofa/engine/executor.mojo:185-191, 555-609)."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class GroupView:
    """One cache group as the kernels see it during a step."""

    page_size: int
    window: int  # 0 = all keys
    max_blocks: int
    block_table: torch.Tensor = None  # int32 [n_seqs, max_blocks]
    slot_map: torch.Tensor = None  # int32 [n_tokens]: cache slot each row is written to


@dataclass
class Layout:
    """Offsets (in int32 words) of every field in the metadata buffer."""

    n_tokens: int
    n_seqs: int
    n_out: int
    fields: dict = field(default_factory=dict)
    total: int = 0

    @staticmethod
    def make(n_tokens: int, n_seqs: int, n_out: int, groups: list) -> "Layout":
        lay = Layout(n_tokens, n_seqs, n_out)
        at = 0

        def add(name, count):
            nonlocal at
            lay.fields[name] = (at, count)
            at += (count + 3) // 4 * 4  # 16-byte aligned fields

        add("token_ids", n_tokens)
        add("token_src", n_tokens)  # -1: the id above; r >= 0: row r of the tokens the step before sampled
        add("positions", n_tokens)
        add("seq_of_token", n_tokens)
        add("q_start", n_seqs + 1)
        add("kv_len", n_seqs)
        add("state_slots", n_seqs)
        add("logit_rows", n_out)
        add("temperature", n_out)  # float32 bits
        add("uniform", n_out)  # float32 bits
        for gi, g in enumerate(groups):
            add(f"slot_map{gi}", n_tokens)
            add(f"block_table{gi}", n_seqs * g.max_blocks)
        lay.total = at
        return lay


@dataclass
class Pending:
    """The residual stream ``h`` is not up to date in its own tensor: its last
    complete value lies in ``base`` (``h`` itself or its alternate buffer), and
    on top of it come the split sums a product left as planes (``partial``) or
    the fixed-point accumulator number ``acc`` that products added into."""

    h: torch.Tensor
    base: torch.Tensor
    partial: object = None
    acc: int = None


class StepContext:
    """Per-step batch description plus scratch allocation."""

    def __init__(self, rt, layout: Layout, dev_meta: torch.Tensor, host_meta: np.ndarray, groups: list, status: torch.Tensor, arena):
        self.rt = rt
        self.arena = arena
        self.layout = layout
        self.n_tokens, self.n_seqs, self.n_out = layout.n_tokens, layout.n_seqs, layout.n_out
        self.host = host_meta
        self.status = status

        def view(name):
            at, count = layout.fields[name]
            return dev_meta[at : at + count]

        self.token_ids = view("token_ids")
        self.token_src = view("token_src")
        self.fed_tokens = None  # int32 on the device: the tokens the step before sampled (set by the step runner)
        self.positions = view("positions")
        self.seq_of_token = view("seq_of_token")
        self.q_start = view("q_start")
        self.kv_len = view("kv_len")
        self.state_slots = view("state_slots")
        self.logit_rows = view("logit_rows")
        self.temperature = view("temperature").view(torch.float32)
        self.uniform = view("uniform").view(torch.float32)
        self.groups = []
        for gi, g in enumerate(groups):
            gv = GroupView(g.page_size, g.window, g.max_blocks)
            gv.slot_map = view(f"slot_map{gi}")
            gv.block_table = view(f"block_table{gi}").view(layout.n_seqs, g.max_blocks)
            self.groups.append(gv)
        # host-side facts parts may branch on (never read back from the device)
        self.max_q_len = 0
        self.max_kv_len = 0
        self.decode_only = False
        self.max_context = 0  # the longest a request may ever get
        self.capturing = False  # the step is being recorded as a CUDA graph: launch shapes must not depend on this step's lengths

        self.any_hot = True  # some wanted row samples with a positive temperature
        self.pending = None  # a Pending: what the residual stream's own tensor still lacks
        # Small decode steps keep the stream as base + fixed-point accumulator (see open_stream)
        self.stream_acc = None  # int64 [2, rows, hidden], given by the step runner; both zero between steps
        self._stream = None

    # -- the residual stream ---------------------------------------------------------------------
    # A product that adds into the stream may leave its split sums for the next reader to add
    # (planes, ``set_pending``), and in decode steps of a few tokens it adds them into one of two
    # 64-bit fixed-point accumulators instead (``accumulator_for`` / ``owe_accumulator``): integer
    # adds give the same sum in any order.  The product that reads the stream next (q/k/v, gate/up)
    # then makes its operand from base + accumulator, norm included, writes the sum to the stream's
    # other buffer (which becomes the base) and clears the accumulator that was not read; readers
    # that cannot do that get the stream settled in its own tensor first.
    def open_stream(self, h) -> None:
        """Called by the model once ``h`` exists: steps of few enough tokens
        for the runner's accumulators, in bfloat16, keep ``h`` as base +
        accumulator."""
        acc = self.stream_acc
        if acc is None or self.n_tokens > acc.shape[1] or h.shape[1] != acc.shape[2] or h.shape[1] % 8 or self.rt.dtype != torch.bfloat16:
            return
        self._stream = {"h": h, "alt": self.buf(tuple(h.shape), torch.float32), "acc": [acc[0, : self.n_tokens], acc[1, : self.n_tokens]], "next": 0, "unclean": set()}

    def stream_of(self, h):
        return self._stream if self._stream is not None and self._stream["h"] is h else None

    def accumulator_for(self, h):
        """The accumulator a product that adds into ``h`` should add into, or
        None when the stream is kept whole (the product then adds in place or
        leaves planes)."""
        st = self.stream_of(h)
        if st is None or (self.pending is not None and (self.pending.partial is not None or self.pending.acc is not None)):
            return None
        return st["acc"][st["next"]]

    def owe_accumulator(self, h) -> None:
        """A product has added into ``accumulator_for(h)``."""
        st = self.stream_of(h)
        base = self.pending.base if self.pending is not None else h
        self.pending = Pending(h, base, None, st["next"])
        st["unclean"].add(st["next"])

    def stream_read(self, h, new_base, pend) -> None:
        """A product has read the stream as base + accumulator and written the
        sum to ``new_base``; it cleared the accumulator it did not read."""
        st = self.stream_of(h)
        if pend is not None and pend.acc is not None:
            st["next"] = 1 - pend.acc
            st["unclean"].discard(1 - pend.acc)
        self.pending = Pending(h, new_base) if new_base is not h else None

    def other_base(self, h, base):
        st = self.stream_of(h)
        return st["alt"] if base is h else h

    def set_pending(self, h, partial) -> None:
        """A product into the residual stream ``h`` left partial sums behind;
        the next reader of ``h`` adds them (norms do it while they read)."""
        if self.pending is not None and self.pending.h is h and self.pending.partial is None and self.pending.acc is None:
            self.pending = Pending(h, self.pending.base, partial)  # the base had moved, nothing else was owed
            return
        self.flush_pending()
        self.pending = Pending(h, h, partial)

    def take_pending(self, h):
        """What ``h`` still lacks (a :class:`Pending`), handing over the duty
        to bring it up to date; None when it is complete."""
        if self.pending is not None and self.pending.h is h:
            pend = self.pending
            self.pending = None
            return pend
        return None

    def accumulators(self, h, pend):
        """(the accumulator ``pend`` owes, the other one) as tensors, for a
        reader that adds the first to the stream and leaves both zero."""
        st = self.stream_of(h)
        st["unclean"].clear()
        return st["acc"][pend.acc], st["acc"][1 - pend.acc]

    def flush_pending(self) -> None:
        """Bring the residual stream up to date in its own tensor now."""
        if self.pending is None:
            return
        from ..csrc import ops

        pend = self.pending
        self.pending = None
        h = pend.h
        if pend.acc is not None:
            acc, other = self.accumulators(h, pend)
            ops.stream_settle(h, pend.base, acc, other)
        elif pend.base is not h:
            h.copy_(pend.base)
        if pend.partial is not None:
            ops.splitk_reduce(h, pend.partial.sums, pend.partial.bias, pend.partial.splits, ops.EPI_RESIDUAL)

    def close_stream(self) -> None:
        """The step's last reader of the stream is done: what is still owed is
        dropped, and an accumulator that nobody left zero is cleared (both are
        zero between steps)."""
        self.pending = None
        if self._stream is not None:
            for i in sorted(self._stream["unclean"]):
                self._stream["acc"][i].zero_()
            self._stream["unclean"].clear()

    def host_field(self, name: str) -> np.ndarray:
        at, count = self.layout.fields[name]
        return self.host[at : at + count]

    def buf(self, shape, dtype) -> torch.Tensor:
        """Scratch for this step (uninitialised): a slice of the step runner's
        arena, nothing is allocated.  Inside a layer it is valid until the
        layer after the next begins, outside until the step ends."""
        return self.arena.buf(shape, dtype)

    def begin_layer(self) -> None:
        """The model calls this before each entry of its run list."""
        self.arena.begin_layer()

    def end_layers(self) -> None:
        self.arena.end_layers()
