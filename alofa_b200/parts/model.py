"""A whole model put together from a :class:`~alofa_b200.config.spec.ModelSpec`.

The run list is data: ``spec.run`` names, per position, which layer runs and
which cache it uses.  A layer named twice runs twice with the same weights; an
entry whose cache is an earlier entry's reads that cache and writes nothing
(layer order of the one shipped architecture: src/alofa/model/arch/qwen.mojo:1367-1372)."""
from __future__ import annotations

import numpy as np
import torch

from ..config.spec import ModelSpec
from .base import Runtime, build_part


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.embedding = build_part("embedding", spec.embedding, rt)
        self.layers = [build_part("block", layer.block, rt) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, rt)
        self.head = build_part("head", spec.head, rt)
        self.run = [(e.layer, i if e.cache is None else e.cache) for i, e in enumerate(spec.run)]

    def parts(self):
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def tensors(self) -> dict:
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state: dict) -> None:
        state = dict(state)
        for part in self.parts():
            part.load(state)

    def graph_safe(self) -> bool:
        """True when every part may be recorded in a CUDA graph."""
        return all(part.graph_safe for part in self.parts())

    def scratch_row_bytes(self) -> tuple:
        """(bytes per token that live for a whole step, bytes per token of the
        layer that needs most): what the step runner sizes its arena from."""
        hidden = self.spec.hidden_size
        per_layer = max([getattr(block, "scratch_row_bytes", lambda: 0)() for block in self.layers] + [8 * hidden])
        return 4 * hidden + 4 * hidden, per_layer

    def cache_plan(self) -> dict:
        """run index -> cache spec, for the entries that own a cache."""
        return {i: self.layers[layer].cache_spec() for i, (layer, cache) in enumerate(self.run) if cache == i}

    def forward(self, ctx, caches: dict) -> torch.Tensor:
        """Logits (fp32) at ``ctx.logit_rows`` for the step's tokens (None when
        no row is wanted; the final norm and the head run on wanted rows only)."""
        h = ctx.buf((ctx.n_tokens, self.spec.hidden_size), torch.float32)
        ctx.open_stream(h)
        self.embedding.forward(ctx, h)
        for i, (layer, cache) in enumerate(self.run):
            block = self.layers[layer]
            if not getattr(block, "absorbs_pending", False):
                ctx.flush_pending()
            ctx.begin_layer()
            block.forward(ctx, h, caches.get(cache), writes=(cache == i))
        ctx.end_layers()
        if ctx.n_out == 0:  # a prompt portion whose logits nobody wants
            ctx.close_stream()
            return None
        if not getattr(self.final_norm, "absorbs_pending", False):
            ctx.flush_pending()
        # every row wanted, in order (a decode step): no picking, and a norm that reads the stream as base + accumulator may
        rows = ctx.logit_rows
        if ctx.n_out == ctx.n_tokens and bool((ctx.host_field("logit_rows") == np.arange(ctx.n_tokens, dtype=np.int32)).all()):
            rows = None
        x = self.final_norm.forward(ctx, h, rows)
        ctx.close_stream()
        return self.head.forward(ctx, x)

def expected_tensors(spec: ModelSpec) -> dict:
    """name -> TensorSpec of everything the model reads from a checkpoint."""
    return Model(spec, Runtime(torch.device("cpu"), torch.float32)).tensors()
