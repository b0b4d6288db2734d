"""How one layer arranges its parts.

``prenorm_residual``: ``h += mixer(norm_a(h)); h += feed_forward(norm_b(h))``
(src/alofa/model/arch/qwen.mojo:1367-1372, 1418-1510).  The residual stream
``h`` is fp32; the parts add into it."""
from __future__ import annotations

from .base import Part, build_part, register_part


class PrenormResidual(Part):
    family = "block"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer = build_part("mixer", self.param("mixer"), rt)
        self.feed_forward = build_part("feed_forward", self.param("feed_forward"), rt)
        self.mixer_norm = build_part("norm", self.param("mixer_norm"), rt)
        self.feed_forward_norm = build_part("norm", self.param("feed_forward_norm"), rt)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensors(self):
        out = {}
        for part in self.parts():
            out.update(part.tensors())
        return out

    def load(self, state):
        for part in self.parts():
            part.load(state)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def scratch_row_bytes(self) -> int:
        return sum(getattr(part, "scratch_row_bytes", lambda: 0)() for part in self.parts())

    absorbs_pending = True  # its norms add partial sums owed to h; other readers get them flushed first

    def _norm(self, norm, ctx, h, reader):
        if not getattr(norm, "absorbs_pending", False):
            ctx.flush_pending()
            return norm.forward(ctx, h)
        # a reader that says so may get rows still to be made (the norm folded into its own product)
        if getattr(reader, "takes_normed_rows", False) and getattr(norm, "gives_normed_rows", False):
            return norm.forward(ctx, h, lazy=True)
        return norm.forward(ctx, h)

    def forward(self, ctx, h, cache, writes=True):
        x = self._norm(self.mixer_norm, ctx, h, self.mixer)
        self.mixer.forward(ctx, x, h, cache, writes)
        x = self._norm(self.feed_forward_norm, ctx, h, self.feed_forward)
        self.feed_forward.forward(ctx, x, h)


register_part("block", "prenorm_residual", PrenormResidual)
