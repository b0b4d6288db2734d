"""The step function: a batch of (request, its next tokens) in, logits at the
wanted places out.

A step runs only the tokens it is given, as one batch, from the cache that
earlier steps left: portions of prompts beside single decoded tokens, cut
anywhere.  It reserves pages for the new tokens and fills the step's metadata
(one native call into the cache manager), copies the metadata to the device
once, runs the model, and then tells the cache manager that the entries are
written (which gives back pages behind windows).  Which requests run, and with
how many tokens, is decided above it (scheduler, trace replay).  The
reference's counterpart is ``BatchExecutor.plan`` + ``forward``
(src/alofa/engine/executor.mojo:555-859).

Steps that hold one token per request and want every row (plain decoding) are
replayed as CUDA graphs, one graph per batch size: the metadata buffer has the
same layout and address every time, so a replay only needs the new metadata.
Steps with prompt portions are recorded too, once a shape (tokens, requests,
wanted rows) comes a third time; a few such graphs are kept."""
from __future__ import annotations

from dataclasses import dataclass
import os
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, GroupSpec
from ..cache.storage import CacheStorage, group_windows
from ..csrc import ops
from ..errors import AlofaError
from ..parts.base import PagedKV
from ..parts.model import Model
from .arena import Arena
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
    feed: int = -1  # >= 0: the (one) token is row `feed` of what the step before sampled; `tokens` holds a placeholder


@dataclass
class DecodeGraph:
    graph: "torch.cuda.CUDAGraph"
    logits: Optional[torch.Tensor]
    tokens: Optional[torch.Tensor]
    kernels: int


class StepRunner:
    """Owns the caches of one model and runs steps over them."""

    # Decode steps of up to this many tokens keep the residual stream as base + accumulator: the
    # products into the stream add their split sums with integer atomics and the norm after them
    # reads 12 bytes an element instead of one plane per split (batch 64: 1.49 -> 1.45 ms per step).
    STREAM_TOKENS = 64

    def __init__(self, model: Model, block_size: int, num_pages, max_requests: int, max_tokens: int, max_step_tokens: int, cuda_graphs: bool = True):
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
        on_gpu = self.rt.device.type == "cuda"
        self._dev_meta = torch.zeros(words, dtype=torch.int32, device=self.rt.device)
        self._host_meta = [torch.zeros(words, dtype=torch.int32).pin_memory() if on_gpu else torch.zeros(words, dtype=torch.int32) for _ in range(2)]
        self._host_event = [None, None]
        self._flip = 0
        self._status = torch.zeros(1, dtype=torch.int32, device=self.rt.device)
        # the tokens of the last sampled step stay here, where the next step's embedding can read them
        self._fed = torch.zeros(max(max_step_tokens, 1), dtype=torch.int32, device=self.rt.device)
        self.feeds_tokens = bool(getattr(model.embedding, "reads_fed_tokens", False))
        # Scratch of every step: sized once here for the largest step (its rows' longest-lived
        # buffers, one row of logits per request) and handed out as slices; nothing is allocated per step.
        step_row, layer_row = model.scratch_row_bytes()
        vocab_bytes = 4 * model.spec.vocab_size
        self.arena = Arena(self.rt.device, max_step_tokens * step_row + max_requests * vocab_bytes * 5 // 4 + (1 << 20),
                           max_step_tokens * layer_row * 5 // 4 + (4 << 20))
        # Decode steps of up to STREAM_TOKENS tokens keep the residual stream as a base tensor plus one
        # of two fixed-point accumulators that the products add into (see StepContext.open_stream); both
        # are zero between steps.  ALOFA_STREAM_ACC=0 keeps the stream in one tensor, as larger steps do.
        self._stream_acc = None
        if on_gpu and self.rt.dtype == torch.bfloat16 and os.environ.get("ALOFA_STREAM_ACC", "1") != "0":
            self._stream_acc = torch.zeros((2, self.STREAM_TOKENS, model.spec.hidden_size), dtype=torch.int64, device=self.rt.device)
        self._layouts = {}
        self.cuda_graphs = cuda_graphs and on_gpu and model.graph_safe()
        self._graphs = {}  # decode steps by batch size; steps with prompt portions by (tokens, requests, wanted rows)
        self.prompt_graphs = self.cuda_graphs and os.environ.get("ALOFA_PROMPT_GRAPHS", "1") != "0"
        self.max_prompt_graphs = 4
        self._seen_shapes = {}

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
    def _layout(self, n_tokens: int, n_seqs: int, n_out: int):
        key = (n_tokens, n_seqs, n_out)
        hit = self._layouts.get(key)
        if hit is None:
            lay = Layout.make(n_tokens, n_seqs, n_out, self._group_shapes)
            names = ["positions", "seq_of_token", "q_start", "kv_len", "state_slots", "logit_rows"]
            for gi in range(len(self._group_shapes)):
                names += [f"slot_map{gi}", f"block_table{gi}"]
            offsets = np.array([lay.fields[n][0] for n in names], dtype=np.int32)
            hit = (lay, offsets)
            if len(self._layouts) < 4096:
                self._layouts[key] = hit
        return hit

    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve pages and fill the step's metadata (host and device)."""
        n_seqs = len(entries)
        if n_seqs == 0:
            raise AlofaError("invalid_argument", "nothing was planned for this step")
        slots = np.fromiter((e.slot for e in entries), dtype=np.int32, count=n_seqs)
        counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=n_seqs)
        want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=n_seqs)
        n_tokens, n_out = int(counts.sum()), int(want_counts.sum())
        if counts.min() <= 0:
            raise AlofaError("invalid_argument", "a step entry has no tokens")
        if n_tokens > self.max_step_tokens or n_seqs > self.max_requests:
            raise AlofaError("capacity", "the step is larger than the engine was built for", f"tokens={n_tokens} max={self.max_step_tokens} requests={n_seqs} max={self.max_requests}")
        if len(set(slots.tolist())) != n_seqs:
            raise AlofaError("invalid_argument", "a request appears twice in one step")
        if n_tokens == n_seqs:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=n_seqs)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= self.model.spec.vocab_size:
            raise AlofaError("out_of_range", "token id outside the vocabulary", f"vocab={self.model.spec.vocab_size}")
        for e, n in zip(entries, counts):
            have = self.manager.computed_len(e.slot)
            if have + n > self.max_tokens:
                raise AlofaError("out_of_range", "history would outgrow the context window", f"slot={e.slot} have={have} add={n} max_tokens={self.max_tokens}")
        if n_out == n_seqs and n_tokens == n_seqs:
            wants = np.zeros(n_seqs, dtype=np.int32)
        elif n_out:
            wants = np.concatenate([np.asarray(e.want, dtype=np.int32) for e in entries if len(e.want)])
        else:
            wants = np.zeros(1, dtype=np.int32)

        layout, offsets = self._layout(n_tokens, n_seqs, n_out)
        flip = self._flip
        self._flip ^= 1
        if self._host_event[flip] is not None:
            self._host_event[flip].synchronize()
        host_t = self._host_meta[flip]
        host = host_t.numpy()
        at, n = layout.fields["token_ids"]
        host[at : at + n] = tokens
        at, n = layout.fields["token_src"]
        host[at : at + n] = -1
        if self.feeds_tokens:
            row = 0
            for e, count in zip(entries, counts):
                if e.feed >= 0:
                    if count != 1:
                        raise AlofaError("invalid_argument", "a fed-back token stands alone in its entry")
                    host[at + row] = e.feed
                row += int(count)
        if n_out:
            at, n = layout.fields["temperature"]
            host[at : at + n].view(np.float32)[:] = np.repeat(np.fromiter((e.temperature for e in entries), dtype=np.float32, count=n_seqs), want_counts)
            at, n = layout.fields["uniform"]
            host[at : at + n].view(np.float32)[:] = np.repeat(np.fromiter((e.uniform for e in entries), dtype=np.float32, count=n_seqs), want_counts)
        max_q, max_kv, _ = self.manager.plan_step(slots, counts, want_counts, wants, host_t.data_ptr(), offsets, self.manager.max_blocks)
        self._dev_meta[: layout.total].copy_(host_t[: layout.total], non_blocking=True)
        if self.rt.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._host_event[flip] = ev
        ctx = StepContext(self.rt, layout, self._dev_meta, host, self._group_shapes, self._status, self.arena)
        self.arena.begin_step()
        ctx.fed_tokens = self._fed if self.feeds_tokens else None
        ctx.stream_acc = self._stream_acc
        ctx.max_q_len, ctx.max_kv_len = max_q, max_kv
        ctx.decode_only = max_q == 1
        ctx.max_context = self.max_tokens
        ctx.slots, ctx.counts = slots, counts
        ctx.any_hot = any(e.temperature > 0.0 for e in entries)
        return ctx

    def commit(self, ctx: StepContext) -> None:
        """The step's entries are written: advance the cache manager."""
        self.manager.commit_step(ctx.slots, ctx.counts)

    def _context_bucket(self, longest: int) -> int:
        """Decode graphs are recorded per batch size and per bucket of the
        longest context in the step (powers of two): the number of key splits
        that attention launches inside a graph then follows the real lengths
        instead of the longest context the engine allows."""
        bucket = 256
        while bucket < longest:
            bucket *= 2
        return min(bucket, max(self.max_tokens, 1))

    def _run(self, ctx: StepContext, sample: bool):
        """(logits or None, tokens or None) for a prepared step."""
        if self.cuda_graphs and ctx.decode_only and ctx.n_out == ctx.n_seqs:
            ctx.max_context = self._context_bucket(ctx.max_kv_len)
            key = (ctx.n_seqs, ctx.max_context, "decode")
            g = self._graphs.get(key)
            if g is None:
                return self._capture(ctx, key, sample)
            g.graph.replay()
            ops.count_launches(g.kernels)
            return g.logits, g.tokens
        if self.prompt_graphs and not ctx.decode_only:
            # A step with prompt portions is some two hundred launches, about as long to issue from
            # Python as to run: a shape (tokens, requests, wanted rows) met a third time is recorded
            # and replayed from then on.  A few shapes are kept, the least recently used one goes.
            key = (ctx.n_tokens, ctx.n_seqs, ctx.n_out)
            g = self._graphs.pop(key, None)
            if g is None:
                seen = self._seen_shapes.get(key, 0)
                if len(self._seen_shapes) > 4096:
                    self._seen_shapes.clear()
                self._seen_shapes[key] = seen + 1
                if seen >= 2:
                    kept = [k for k in self._graphs if len(k) == 3 and k[2] != "decode"]
                    if len(kept) >= self.max_prompt_graphs:
                        del self._graphs[kept[0]]
                    logits, tokens = self._capture(ctx, key, sample)
                    self._graphs[key] = self._graphs.pop(key)  # most recently used last
                    return (logits if ctx.n_out else None), (tokens if ctx.n_out else None)
            if g is not None:
                self._graphs[key] = g  # most recently used last
                g.graph.replay()
                ops.count_launches(g.kernels)
                return (g.logits if ctx.n_out else None), (g.tokens if ctx.n_out else None)
        with ops.bound_stream():
            logits = self.model.forward(ctx, self.storage.caches)
            tokens = None
            if sample and logits is not None:
                tokens = self._sample(ctx, logits, ctx.any_hot)
        return logits, tokens

    def _sample(self, ctx: StepContext, logits: torch.Tensor, any_hot: bool) -> torch.Tensor:
        """One token per wanted row by temperature alone (0 = the largest logit),
        left where the next step can take them as its input."""
        tokens = self._fed[: ctx.n_out]
        scratch = ctx.buf((2 * ctx.n_out * ops.ARGMAX_PARTS,), torch.float32)
        ops.sample(tokens, logits, ctx.temperature, ctx.uniform, scratch, any_hot)
        return tokens

    def _capture(self, ctx: StepContext, key, sample: bool):
        """Run the step outright and record it as a CUDA graph for the next
        time its shape comes; returns this run's (logits, tokens).  The step is
        executed once only: recording launches nothing, and the recorded graph
        is first replayed by the NEXT step of this shape, so a part that
        updates per-request state in place advances it once per step.  The
        outright run also loads every kernel before recording and makes the
        arena grow, if it has to, outside the recording; both passes rewind the
        arena first, so they get the same addresses.  Launch shapes inside must
        depend on the shape alone: attention is sized for the bucket of the
        longest context, and in steps with prompt portions for one request
        holding all tokens but one each of the others."""
        ctx.capturing = True
        if not ctx.decode_only:
            ctx.max_q_len = ctx.n_tokens - ctx.n_seqs + 1
        with ops.bound_stream():
            self.arena.begin_step()
            first_logits = self.model.forward(ctx, self.storage.caches)
            first_tokens = self._sample(ctx, first_logits, ctx.any_hot) if (sample and first_logits is not None) else None
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        grown = self.arena.grown
        with torch.cuda.graph(graph), ops.bound_stream():
            self.arena.begin_step()
            logits = self.model.forward(ctx, self.storage.caches)
            tokens = self._sample(ctx, logits, True) if logits is not None else None  # a replay may meet rows of any temperature
        if self.arena.grown != grown or (logits is not None and logits.data_ptr() != first_logits.data_ptr()):
            raise AlofaError("state", "recording a step asked the arena for other memory than running it did")
        self._graphs[key] = DecodeGraph(graph, logits, tokens, ops.launch_count() - before)
        return first_logits, first_tokens

    def forward(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step; logits (fp32, on the device) at the wanted places in
        the order of the entries and of their ``want``, or None if none.  The
        tensor is valid until the next step."""
        ctx = self.prepare(entries)
        logits, _ = self._run(ctx, sample=False)
        self.commit(ctx)
        return logits if ctx.n_out else None

    def forward_logits(self, entries: Sequence[StepEntry]):
        """Run one step; (context, logits or None) for a sampler to use."""
        ctx = self.prepare(entries)
        logits, _ = self._run(ctx, sample=False)
        self.commit(ctx)
        return ctx, (logits if ctx.n_out else None)

    def forward_sampled(self, entries: Sequence[StepEntry]):
        """Run one step and pick a token at every wanted place by temperature
        alone: (context, logits, tokens int32 on the device)."""
        ctx = self.prepare(entries)
        logits, tokens = self._run(ctx, sample=True)
        self.commit(ctx)
        return ctx, logits, tokens

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input since the last check (reads the
        device, so it waits for the stream)."""
        self.raise_status(int(self._status.item()))

    def copy_status(self, host: torch.Tensor) -> None:
        """Queue a copy of the status word into ``host`` (pinned, int32 [1])
        behind the work already on the stream; the caller reads it once an
        event recorded after this call has passed and hands the value to
        :meth:`raise_status`."""
        host.copy_(self._status, non_blocking=True)

    def raise_status(self, code: int) -> None:
        """Turn a status word read from the device into the error it stands
        for; the word is cleared so that the next step starts clean."""
        if code == 0:
            return
        self._status.zero_()
        if self._stream_acc is not None:
            self._stream_acc.zero_()  # a kernel that gave up may have left the step half done
        if code == 2:
            raise AlofaError("state", "a kernel gave up waiting on its own pipeline")
        raise AlofaError("out_of_range", "a kernel met a token id outside the vocabulary")
