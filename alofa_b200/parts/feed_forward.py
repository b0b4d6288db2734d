"""Dense gated feed-forward: ``h += (act(x Wg^T) * (x Wu^T)) Wd^T`` with
``silu(z) = z / (1 + exp(-z))``, no biases
(src/alofa/model/arch/qwen.mojo:1481-1510; src/alofa/kernels/cpu/scalar.mojo:208-231).
The gate and up weights are stacked at load so that one product with a fused
epilogue writes ``silu(gate) * up`` directly."""
from __future__ import annotations

import torch

from ..errors import AlofaError
from .base import Part, TensorSpec, register_part
from .linear import GATED, RESIDUAL, Linear, add_into_stream


class GatedMLP(Part):
    family = "feed_forward"
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        act = self.param("activation", "silu")
        if act != "silu":
            raise AlofaError("unsupported", "gated_mlp supports the silu activation only", f"activation={act}")
        self.gate_up = self.down = None

    def tensors(self):
        pre = self.prefix
        return {
            pre + "gate_proj.weight": TensorSpec((self.inter, self.hidden)),
            pre + "up_proj.weight": TensorSpec((self.inter, self.hidden)),
            pre + "down_proj.weight": TensorSpec((self.hidden, self.inter)),
        }

    def load(self, state):
        pre = self.prefix
        self.gate_up = Linear(torch.cat([state[pre + "gate_proj.weight"], state[pre + "up_proj.weight"]], dim=0), None, GATED)
        self.down = Linear(state[pre + "down_proj.weight"], None, RESIDUAL)

    def scratch_row_bytes(self) -> int:
        return 4 * self.inter + 2 * 4 * self.hidden  # the activation, and the down product's depth split in two

    takes_normed_rows = True  # ``x`` may be rows still to be made: the gate/up product folds the norm in

    def forward(self, ctx, x, h):
        act = ctx.buf((x.shape[0], self.inter), self.rt.dtype)
        self.gate_up(act, x, buf=ctx.buf)
        add_into_stream(ctx, self.down, h, act)


register_part("feed_forward", "gated_mlp", GatedMLP)
