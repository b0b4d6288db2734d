"""Settings of the engine itself, all decided at run time.

The names follow the reference's scheduler configuration
(src/alofa/engine/scheduler.mojo:139-192: token_budget, max_chunk,
block_size, capacity_blocks, watermark_permille, max_wait_ticks) and its
server settings (src/alofa/srv/config.mojo:73-107: max_tokens = context
window per request, max_prompt_tokens, seed); where the reference fixes a
size at compile time (8 requests, 64 rows per step) the size is a field."""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import AlofaError


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"  # "bfloat16" or "float32"
    block_size: int = 64  # tokens per cache page
    capacity_blocks: int = 0  # pages per cache group; 0 = derive from max_batch * max_tokens
    max_batch: int = 64  # live requests
    max_tokens: int = 4096  # context window per request (prompt + generated)
    token_budget: int = 2112  # tokens per step, prefill and decode together
    max_chunk: int = 2048  # longest prompt portion per request per step
    watermark_permille: int = 1000  # occupancy above which running requests are preempted
    max_wait_ticks: int = 8  # ticks after which a waiting request jumps the queue
    seed: int = 1234  # default sampling seed
    cuda_graphs: bool = True  # replay decode-only steps as CUDA graphs
    overlap_steps: bool = True  # launch a step before the host has read the tokens of the one before (they are fed on the device)

    def validate(self) -> None:
        def need(ok, what, detail):
            if not ok:
                raise AlofaError("invalid_argument", what, detail)

        need(self.dtype in ("bfloat16", "float32"), "dtype must be bfloat16 or float32", f"dtype={self.dtype}")
        need(self.block_size > 0 and self.block_size % 16 == 0, "block_size must be a positive multiple of 16", f"block_size={self.block_size}")
        need(self.capacity_blocks >= 0, "capacity_blocks must not be negative", f"capacity_blocks={self.capacity_blocks}")
        need(self.max_batch > 0, "max_batch must be positive", f"max_batch={self.max_batch}")
        need(self.max_tokens > 0, "max_tokens must be positive", f"max_tokens={self.max_tokens}")
        need(self.max_chunk > 0, "max_chunk must be positive", f"max_chunk={self.max_chunk}")
        need(self.token_budget >= 1, "token_budget must be at least one token a step", f"token_budget={self.token_budget}")
        need(0 <= self.watermark_permille <= 1000, "watermark_permille out of range", f"watermark_permille={self.watermark_permille}")
        need(self.max_wait_ticks >= 0, "max_wait_ticks must not be negative", f"max_wait_ticks={self.max_wait_ticks}")
