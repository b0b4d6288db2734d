"""The architecture-neutral description that a model configuration is turned
into: which parts make up each layer, with which sizes and constants, and in
which order the layers run.

Everything here is plain data.  A part is named by ``kind`` (a key of the part
registries in :mod:`alofa_b200.parts`) and carries its sizes in ``params``;
nothing in a spec refers to the architecture it came from, so parts never
learn which model they are in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class PartSpec:
    """One part: ``kind`` chooses the implementation, ``params`` its sizes and
    constants, ``prefix`` the leading part of its tensor names."""

    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass
class LayerSpec:
    """One layer: the arrangement (``block``) and the parts it arranges.  The
    block's params name its mixer, feed-forward and norms as PartSpecs."""

    block: PartSpec


@dataclass
class RunEntry:
    """One position of the run list.

    ``layer`` indexes :attr:`ModelSpec.layers`; a layer may appear more than
    once.  ``cache`` names the cache this run of the layer uses: the index of
    the run entry that owns (writes) it.  An entry whose ``cache`` equals its
    own index owns a fresh cache; an entry that names an earlier index reads
    that entry's cache and writes nothing to it."""

    layer: int
    cache: Optional[int] = None


@dataclass
class ModelSpec:
    """A whole model as data."""

    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: list
    run: list
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        from ..errors import AlofaError

        for i, entry in enumerate(self.run):
            if not 0 <= entry.layer < len(self.layers):
                raise AlofaError("invalid_argument", "run list names a layer that does not exist", f"entry={i} layer={entry.layer}")
            cache = i if entry.cache is None else entry.cache
            if cache > i or cache < 0:
                raise AlofaError("invalid_argument", "a run entry may only read the cache of an earlier entry", f"entry={i} cache={cache}")
            if cache != i:
                owner = self.run[cache]
                if (owner.cache if owner.cache is not None else cache) != cache:
                    raise AlofaError("invalid_argument", "a run entry reads a cache from an entry that does not own one", f"entry={i} cache={cache}")
