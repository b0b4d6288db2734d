"""Token embedding and the output head.

``h[r] = embed[id_r]`` with ids outside the vocabulary refused
(src/alofa/model/arch/qwen.mojo:1391-1413).  The head multiplies the normed
rows whose logits are wanted by ``lm_head.weight`` if the file has it, else by
the embedding when the two are tied (qwen.mojo:1077-1089, 1512-1523); a tied
head shares the embedding's memory."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError
from .base import Part, TensorSpec, register_part
from .linear import STORE, Linear


class TokenEmbedding(Part):
    family = "embedding"
    graph_safe = True
    reads_fed_tokens = True  # honours ctx.token_src: a step may be launched before the host has seen its tokens

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight = None

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, state):
        self.weight = state[self.prefix + "weight"]

    def forward(self, ctx, h):
        ops.embed_gather(h, self.weight, ctx.token_ids, ctx.status, ctx.token_src if ctx.fed_tokens is not None else None, ctx.fed_tokens)

class LinearHead(Part):
    family = "head"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.tied_to = self.params.get("tied_to")
        self.linear = None

    def tensors(self):
        return {self.prefix + "weight": TensorSpec((self.vocab, self.hidden), optional=self.tied_to is not None)}

    def load(self, state):
        name = self.prefix + "weight"
        if name in state:
            weight = state[name]
        elif self.tied_to is not None and self.tied_to in state:
            weight = state[self.tied_to]
        else:
            raise AlofaError("invalid_argument", "the model has no output head weight", f"name={name} tied_to={self.tied_to}")
        self.linear = Linear(weight, None, STORE)

    def forward(self, ctx, x):
        logits = ctx.buf((x.shape[0], self.vocab), torch.float32)
        self.linear(logits, x, buf=ctx.buf)
        return logits

register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
