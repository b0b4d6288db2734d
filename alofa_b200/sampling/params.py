"""Sampling settings, with the reference's names, meanings and defaults
(``SampleParams``, src/alofa/runtime/sampler.mojo:93-118), applied in its
order: logit bias, repetition penalty, frequency and presence penalties,
temperature, top-k, top-p, min-p, softmax, inverse-CDF draw
(sampler.mojo:308-481).  ``temperature == 0`` picks the largest logit, ties to
the lowest index."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import AlofaError


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0  # 0 = off; keeps everything >= the k-th largest (ties survive)
    top_p: float = 1.0  # smallest sorted prefix whose probability reaches top_p
    min_p: float = 0.0  # drops p < min_p * p_max
    repetition_penalty: float = 1.0  # per distinct seen token: x<0 ? x*p : x/p
    frequency_penalty: float = 0.0  # x -= f * count
    presence_penalty: float = 0.0  # x -= p for seen tokens
    min_tokens_to_keep: int = 1  # floor for top-p and min-p
    logit_bias: dict = field(default_factory=dict)  # token id -> additive offset, applied first
    seed: int = 1234
    max_new_tokens: int = 16
    stop_token_ids: tuple = ()  # generation ends after one of these is produced

    def validate(self, vocab_size: int) -> None:
        def need(ok, what, detail):
            if not ok:
                raise AlofaError("invalid_argument", what, detail)

        need(self.temperature >= 0.0, "temperature must not be negative", f"temperature={self.temperature}")
        need(self.top_k >= 0, "top_k must not be negative", f"top_k={self.top_k}")
        need(self.top_p > 0.0, "top_p must be positive", f"top_p={self.top_p}")
        need(0.0 <= self.min_p <= 1.0, "min_p must lie in [0, 1]", f"min_p={self.min_p}")
        need(self.repetition_penalty > 0.0, "repetition_penalty must be positive", f"repetition_penalty={self.repetition_penalty}")
        need(self.max_new_tokens > 0, "max_new_tokens must be positive", f"max_new_tokens={self.max_new_tokens}")
        for idx in self.logit_bias:
            if not 0 <= int(idx) < vocab_size:
                raise AlofaError("out_of_range", "bias index is outside the vocabulary", f"index={idx} vocab={vocab_size}")

    def plain(self) -> bool:
        """True when only the temperature shapes the distribution: the fused
        argmax / softmax-draw kernel serves these."""
        return (
            (self.top_k == 0 and self.top_p >= 1.0 and self.min_p == 0.0 or self.temperature == 0.0)
            and self.repetition_penalty == 1.0
            and self.frequency_penalty == 0.0
            and self.presence_penalty == 0.0
            and not self.logit_bias
        )
