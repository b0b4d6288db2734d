"""The step function: a batch of (request, its next tokens) in, logits at the
wanted places out.

A step runs only the tokens it is given, as one batch, from the cache that
earlier steps left: portions of prompts beside single decoded tokens, cut
anywhere.  It reserves pages for the new tokens, fills the step's metadata,
copies it to the device once, runs the model, and then tells the cache manager
that the entries are written (which gives back pages behind windows).  Which
requests run, and with how many tokens, is decided above it (scheduler, trace
replay).  The reference's counterpart is ``BatchExecutor.plan`` + ``forward``
(src/alofa/engine/executor.mojo:555-859)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, GroupSpec
from ..cache.storage import CacheStorage, group_windows
from ..errors import AlofaError
from ..parts.base import PagedKV
from ..parts.model import Model
from .context import GroupView, Layout, StepContext


@dataclass
class StepEntry:
    """One request's share of a step: its state slot, its next tokens, and the
    places among them (0-based) whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    temperature: float = 0.0  # used when the step samples
    uniform: float = 0.0


class StepRunner:
    """Owns the caches of one model and runs steps over them."""

    def __init__(self, model: Model, block_size: int, num_pages, max_requests: int, max_tokens: int, max_step_tokens: int):
        self.model = model
        self.rt = model.rt
        self.block_size = block_size
        self.max_requests = max_requests
        self.max_tokens = min(max_tokens, model.spec.max_position)
        self.max_step_tokens = max_step_tokens
        plan = model.cache_plan()
        windows = group_windows(plan)
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(windows)
        self.group_specs = [GroupSpec(block_size, n, w) for n, w in zip(num_pages, windows)]
        self.manager = CacheManager(self.group_specs, max_requests, self.max_tokens)
        self.storage = CacheStorage(plan, self.group_specs, max_requests, self.rt.dtype, self.rt.device)
        self.has_paged = any(isinstance(s, PagedKV) for s in plan.values())
        mb = self.manager.max_blocks
        self._group_shapes = [GroupView(block_size, g.window or 0, mb) for g in self.group_specs]
        words = Layout.make(max_step_tokens, max_requests, max_step_tokens, self._group_shapes).total
        self._dev_meta = torch.zeros(words, dtype=torch.int32, device=self.rt.device)
        self._host_meta = [torch.zeros(words, dtype=torch.int32).pin_memory() if self.rt.device.type == "cuda" else torch.zeros(words, dtype=torch.int32) for _ in range(2)]
        self._host_event = [None, None]
        self._flip = 0
        self._status = torch.zeros(1, dtype=torch.int32, device=self.rt.device)
        self._table_row = np.zeros(mb, dtype=np.int32)

    # -- requests -----------------------------------------------------------
    def admit(self, request_id: int) -> int:
        slot = self.manager.admit(request_id)
        self.storage.reset_slot(slot)
        return slot

    def release(self, slot: int) -> None:
        self.manager.release(slot)

    def length(self, slot: int) -> int:
        return self.manager.computed_len(slot)

    # -- the step -----------------------------------------------------------
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve pages and fill the step's metadata (host and device)."""
        n_seqs = len(entries)
        n_tokens = sum(len(e.tokens) for e in entries)
        n_out = sum(len(e.want) for e in entries)
        if n_seqs == 0 or n_tokens == 0:
            raise AlofaError("invalid_argument", "nothing was planned for this step")
        if n_tokens > self.max_step_tokens or n_seqs > self.max_requests:
            raise AlofaError("capacity", "the step is larger than the engine was built for", f"tokens={n_tokens} max={self.max_step_tokens} requests={n_seqs} max={self.max_requests}")
        if len({e.slot for e in entries}) != n_seqs:
            raise AlofaError("invalid_argument", "a request appears twice in one step")
        vocab = self.model.spec.vocab_size
        starts = []
        for e in entries:
            if len(e.tokens) == 0:
                raise AlofaError("invalid_argument", "a step entry has no tokens", f"slot={e.slot}")
            start = self.manager.computed_len(e.slot)
            if start + len(e.tokens) > self.max_tokens:
                raise AlofaError("out_of_range", "history would outgrow the context window", f"slot={e.slot} have={start} add={len(e.tokens)} max_tokens={self.max_tokens}")
            starts.append(start)
        reserved = []
        try:
            for e, start in zip(entries, starts):
                self.manager.reserve(e.slot, start + len(e.tokens))
                reserved.append(e)
        except AlofaError:
            raise

        layout = Layout.make(n_tokens, n_seqs, n_out, self._group_shapes)
        flip = self._flip
        self._flip ^= 1
        if self._host_event[flip] is not None:
            self._host_event[flip].synchronize()
        host_t = self._host_meta[flip]
        host = host_t.numpy()
        f = {k: host[at : at + n] for k, (at, n) in layout.fields.items()}
        row = out = 0
        max_q = max_kv = 0
        temp = f["temperature"].view(np.float32)
        unif = f["uniform"].view(np.float32)
        bs = self.block_size
        for si, (e, start) in enumerate(zip(entries, starts)):
            n = len(e.tokens)
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.min() < 0 or toks.max() >= vocab:
                raise AlofaError("out_of_range", "token id outside the vocabulary", f"slot={e.slot} vocab={vocab}")
            f["token_ids"][row : row + n] = toks
            pos = np.arange(start, start + n, dtype=np.int32)
            f["positions"][row : row + n] = pos
            f["seq_of_token"][row : row + n] = si
            f["q_start"][si] = row
            f["kv_len"][si] = start + n
            f["state_slots"][si] = e.slot
            for w in e.want:
                if not 0 <= w < n:
                    raise AlofaError("out_of_range", "wanted place is outside the entry's tokens", f"slot={e.slot} want={w} tokens={n}")
                f["logit_rows"][out] = row + w
                temp[out] = e.temperature
                unif[out] = e.uniform
                out += 1
            for gi, g in enumerate(self._group_shapes):
                table = f[f"block_table{gi}"].reshape(n_seqs, g.max_blocks)[si]
                nb = self.manager.block_table_into(e.slot, gi, self._table_row)
                table[:nb] = self._table_row[:nb]
                table[nb:] = -1
                f[f"slot_map{gi}"][row : row + n] = table[pos // bs] * bs + pos % bs
            row += n
            max_q = max(max_q, n)
            max_kv = max(max_kv, start + n)
        f["q_start"][n_seqs] = row
        dev = self._dev_meta[: layout.total]
        dev.copy_(host_t[: layout.total], non_blocking=True)
        if self.rt.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._host_event[flip] = ev
        ctx = StepContext(self.rt, layout, self._dev_meta, host, self._group_shapes, self._status)
        ctx.max_q_len, ctx.max_kv_len = max_q, max_kv
        ctx.decode_only = max_q == 1
        ctx.entries = entries
        ctx.starts = starts
        return ctx

    def commit(self, ctx: StepContext) -> None:
        """The step's entries are written: advance the cache manager."""
        for e, start in zip(ctx.entries, ctx.starts):
            self.manager.advance(e.slot, start + len(e.tokens))

    def forward(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step; logits (fp32, on the device) at the wanted places in
        the order of the entries and of their ``want``, or None if none."""
        ctx = self.prepare(entries)
        logits = self.model.forward(ctx, self.storage.caches)
        self.commit(ctx)
        return logits if ctx.n_out else None

    def forward_logits(self, entries: Sequence[StepEntry]):
        """Run one step; (context, logits or None) for a sampler to use."""
        ctx = self.prepare(entries)
        logits = self.model.forward(ctx, self.storage.caches)
        self.commit(ctx)
        return ctx, (logits if ctx.n_out else None)

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input since the last check (reads the
        device, so it waits for the stream)."""
        if int(self._status.item()) != 0:
            self._status.zero_()
            raise AlofaError("out_of_range", "a kernel met a token id outside the vocabulary")
