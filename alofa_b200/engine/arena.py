"""Scratch memory of the step function: one arena, nothing allocated per step.

Every buffer a step needs between its kernels (the residual stream, a layer's
activations, split sums, logits) is a slice of memory that the step runner owns
for its whole life, after the reference's executor, which sizes its step
buffers once (src/alofa/engine/executor.mojo:130-145, 611-663).  The arena has
three regions, each a bump allocator that is rewound, not freed:

* ``step``: what lives for the whole step (residual stream, logits);
* two ``layer`` regions used in turn: a layer's buffers are handed out from one
  while the sums that the layer before still owes the residual stream (left in
  the other) are read, and the region is rewound when its turn comes again.
  Consecutive layers thus write the same few megabytes, which stay in L2.

A region is a chain of blocks.  The first block is sized at construction from
the largest step and the model's widest row; should a step need more (a part
nobody sized for, every row's logits wanted), a further block is appended once
and kept, so addresses handed out earlier - those a recorded CUDA graph holds -
stay valid, and a sequence of requests that fitted before gets the same
addresses again."""
from __future__ import annotations

import torch

ALIGN = 256


class Region:
    def __init__(self, device, first_bytes: int):
        self.device = device
        self.blocks = []
        self.block = 0
        self.offset = 0
        self.grown = 0  # blocks appended after construction
        self._append(max(int(first_bytes), ALIGN))
        self.grown = 0

    def _append(self, nbytes: int) -> None:
        nbytes = -(-nbytes // ALIGN) * ALIGN
        self.blocks.append(torch.empty(nbytes, dtype=torch.uint8, device=self.device))
        self.grown += 1

    def rewind(self) -> None:
        self.block = 0
        self.offset = 0

    def take(self, nbytes: int) -> torch.Tensor:
        nbytes = max(-(-int(nbytes) // ALIGN) * ALIGN, ALIGN)
        while True:
            blk = self.blocks[self.block]
            if self.offset + nbytes <= blk.numel():
                out = blk[self.offset : self.offset + nbytes]
                self.offset += nbytes
                return out
            if self.block + 1 == len(self.blocks):
                self._append(max(nbytes, 2 * self.blocks[-1].numel()))
            self.block += 1
            self.offset = 0

    @property
    def bytes(self) -> int:
        return sum(b.numel() for b in self.blocks)


class Arena:
    """``buf(shape, dtype)`` hands out uninitialised device memory that is
    valid until the region it came from is rewound: the end of the step for
    the step region, two layers later for a layer region."""

    def __init__(self, device, step_bytes: int, layer_bytes: int):
        self.device = device
        self.step = Region(device, step_bytes)
        self.layers = [Region(device, layer_bytes), Region(device, layer_bytes)]
        self.current = self.step
        self.turn = 0

    def begin_step(self) -> None:
        self.step.rewind()
        self.layers[0].rewind()
        self.layers[1].rewind()
        self.current = self.step
        self.turn = 0

    def begin_layer(self) -> None:
        """The buffers of the layer before last are dead: reuse their region."""
        self.turn ^= 1
        self.current = self.layers[self.turn]
        self.current.rewind()

    def end_layers(self) -> None:
        self.current = self.step

    def buf(self, shape, dtype) -> torch.Tensor:
        if isinstance(shape, int):
            shape = (shape,)
        count = 1
        for s in shape:
            count *= int(s)
        width = dtype.itemsize
        return self.current.take(count * width)[: count * width].view(dtype).view(*shape)

    @property
    def bytes(self) -> int:
        return self.step.bytes + sum(r.bytes for r in self.layers)

    @property
    def grown(self) -> int:
        return self.step.grown + sum(r.grown for r in self.layers)
