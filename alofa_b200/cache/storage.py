"""Device memory of the caches.

For every run entry that owns a cache the model says what it needs
(:class:`~alofa_b200.parts.base.PagedKV` or
:class:`~alofa_b200.parts.base.SlotState`).  Paged caches are sorted into
groups by their window (all keys, or the last ``window``); a group's page ids
are valid in every layer cache of the group.  A layer cache is two tensors
``k, v: [num_pages * block_size, kv_heads, head_dim]``; cache slot
``page * block_size + offset`` holds one token (the reference keeps
``[layers * blocks, block_size, kv_dim]`` and offsets the block id by the
layer, src/alofa/engine/executor.mojo:117-127, 301-310).  Slot-state caches
are one tensor ``[max_requests, *shape]`` each."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..errors import AlofaError
from ..parts.base import PagedKV, SlotState


@dataclass
class LayerCache:
    """Paged keys and values of one layer cache."""

    group: int
    k: torch.Tensor
    v: torch.Tensor


@dataclass
class StateCache:
    """Fixed-size per-request state of one layer cache: ``state[slot]``."""

    state: torch.Tensor


def group_windows(plan: dict) -> list:
    """The distinct windows of a cache plan, all-keys (None) first; empty when
    no layer wants pages (the model then has state slots only, and neither the
    cache manager nor the scheduler books a page for it)."""
    windows = {spec.window for spec in plan.values() if isinstance(spec, PagedKV)}
    return ([None] if None in windows else []) + sorted(w for w in windows if w is not None)


class CacheStorage:
    def __init__(self, plan: dict, groups: list, max_requests: int, dtype: torch.dtype, device):
        """``plan``: run index -> cache spec (owners only); ``groups``: the
        :class:`GroupSpec` list in the order of :func:`group_windows`."""
        windows = [g.window for g in groups]
        self.groups = groups
        self.caches = {}
        self.bytes = 0
        for idx, spec in plan.items():
            if isinstance(spec, PagedKV):
                if spec.window not in windows:
                    raise AlofaError("invalid_argument", "no cache group for this window", f"window={spec.window} groups={windows}")
                gi = windows.index(spec.window)
                g = groups[gi]
                shape = (g.num_pages * g.block_size, spec.num_kv_heads, spec.head_dim)
                k = torch.zeros(shape, dtype=dtype, device=device)
                v = torch.zeros(shape, dtype=dtype, device=device)
                self.caches[idx] = LayerCache(gi, k, v)
                self.bytes += 2 * k.numel() * k.element_size()
            elif isinstance(spec, SlotState):
                st = torch.zeros((max_requests,) + tuple(spec.shape), dtype=spec.dtype, device=device)
                self.caches[idx] = StateCache(st)
                self.bytes += st.numel() * st.element_size()
            elif spec is not None:
                raise AlofaError("unsupported", "unknown cache spec", f"entry={idx} spec={spec!r}")

    def reset_slot(self, slot: int) -> None:
        """Zero the fixed-size state of a slot when a request starts in it."""
        for cache in self.caches.values():
            if isinstance(cache, StateCache):
                cache.state[slot].zero_()

    @staticmethod
    def bytes_per_token(plan: dict, dtype: torch.dtype) -> dict:
        """window -> bytes of paged cache one token takes in that group."""
        width = torch.empty((), dtype=dtype).element_size()
        out = {}
        for spec in plan.values():
            if isinstance(spec, PagedKV):
                out[spec.window] = out.get(spec.window, 0) + 2 * spec.num_kv_heads * spec.head_dim * width
        return out
