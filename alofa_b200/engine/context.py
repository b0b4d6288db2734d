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
        self.pending = None  # (residual stream, Partial): sums a deferred product still owes it

    def set_pending(self, h, partial) -> None:
        """A product into the residual stream ``h`` left partial sums behind;
        the next reader of ``h`` adds them (norms do it while they read)."""
        self.flush_pending()
        self.pending = (h, partial)

    def take_pending(self, h):
        """The partial sums owed to ``h``, handing over the duty to add them."""
        if self.pending is not None and self.pending[0] is h:
            partial = self.pending[1]
            self.pending = None
            return partial
        return None

    def flush_pending(self) -> None:
        """Add any owed partial sums into their residual stream now."""
        if self.pending is not None:
            from ..csrc import ops

            h, partial = self.pending
            self.pending = None
            ops.splitk_reduce(h, partial.sums, partial.bias, partial.splits, ops.EPI_RESIDUAL)

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
