"""What every part is, and the registries parts are chosen from.

A model is put together from parts of seven families: ``embedding``,
``position`` (position encoding), ``mixer`` (attention here), ``feed_forward``
(dense or routed), ``norm``, ``block`` (how one layer arranges its mixer,
feed-forward and norms) and ``head``.  A part is chosen by the ``kind`` of its
:class:`~alofa_b200.config.spec.PartSpec` and gets its sizes and constants
from the spec's ``params``; it never learns which model it is in.

Interfaces (``ctx`` is the step's :class:`~alofa_b200.engine.context.StepContext`;
``h`` is the fp32 residual stream ``[tokens, hidden]``):

* every part: ``tensors() -> {name: TensorSpec}`` and ``load(state)``;
* norm: ``forward(ctx, h, rows=None) -> x`` in the compute dtype;
* position: ``rotary_table()`` (cos/sin table and rotary_dim, or None) and
  ``apply(ctx, q, k)`` for encodings that are not rotary;
* mixer: ``cache_spec()`` (PagedKV, SlotState or None) and
  ``forward(ctx, x, h, cache, writes)`` which adds its output into ``h``;
* feed_forward: ``forward(ctx, x, h)`` which adds its output into ``h``;
* block: ``cache_spec()`` and ``forward(ctx, h, cache, writes)``;
* embedding: ``forward(ctx, h)`` fills ``h`` from ``ctx.token_ids``;
* head: ``forward(ctx, x) -> logits`` fp32 ``[rows, vocab]``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.spec import PartSpec
from ..errors import AlofaError

FAMILIES = ("embedding", "position", "mixer", "feed_forward", "norm", "block", "head")
_REGISTRY: dict = {f: {} for f in FAMILIES}


@dataclass
class TensorSpec:
    """A tensor a part expects under its name: shape, the law random weights
    are drawn from ("normal": N(0, 0.02); "ones": 1 + N(0, 0.01)), and whether
    the file may leave it out."""

    shape: tuple
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class PagedKV:
    """A mixer's need of a paged key/value cache: ``window`` None = all keys."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotState:
    """A mixer's need of per-request state of fixed size: one tensor of
    ``shape`` and ``dtype`` per live request, zeroed when a request starts."""

    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What parts share: the device and the compute dtype."""

    device: torch.device
    dtype: torch.dtype  # torch.float32 (true 32-bit path) or torch.bfloat16


class Part:
    """Base of all parts.  Constructors only record sizes; device memory is
    touched in :meth:`load`."""

    family = ""
    # True when forward only launches kernels on the current stream with no
    # host-side dependence on device data: such a part can be recorded in a
    # CUDA graph.  Parts must opt in.
    graph_safe = False

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.spec = spec
        self.params = spec.params
        self.prefix = spec.prefix
        self.rt = rt

    def tensors(self) -> dict:
        return {}

    def load(self, state: dict) -> None:
        pass

    def param(self, key, default=None):
        if key not in self.params:
            if default is None:
                raise AlofaError("invalid_argument", "part is missing a parameter", f"kind={self.spec.kind} key={key}")
            return default
        return self.params[key]


def register_part(family: str, kind: str, cls, replace: bool = False) -> None:
    """Make ``cls`` available as ``kind`` of ``family``."""
    if family not in _REGISTRY:
        raise AlofaError("invalid_argument", "unknown part family", f"family={family} known={FAMILIES}")
    if kind in _REGISTRY[family] and not replace:
        raise AlofaError("invalid_argument", "part kind is already registered", f"family={family} kind={kind}")
    _REGISTRY[family][kind] = cls


def build_part(family: str, spec: PartSpec, rt: Runtime):
    kinds = _REGISTRY[family]
    if spec.kind not in kinds:
        raise AlofaError("unsupported", "no part of this kind is registered", f"family={family} kind={spec.kind} known={sorted(kinds)}")
    return kinds[spec.kind](spec, rt)


def as_float32_vector(t: torch.Tensor) -> torch.Tensor:
    """Norm weights and biases are handed to the kernels in fp32 (widening
    bf16 is exact)."""
    return t.to(torch.float32).contiguous()
