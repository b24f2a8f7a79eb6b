"""Per-request generation settings, fixed for the request's lifetime.

Names, defaults and meanings are the reference's `GenerationConfig`
(`engine/src/sampling.rs:80-119`): `temperature <= 0` means greedy and is the
switch (there is no separate mode flag); `top_k` clamps to [1, vocab]
(`:209-220`); the default is greedy with top_k 40 and seed 1234.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

DEFAULT_TEMPERATURE = 0.8      # the command line's default (engine/src/main.rs:486)
DEFAULT_TOP_K = 40
DEFAULT_SEED = 1234
DEFAULT_MAX_TOKENS = 64


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = DEFAULT_MAX_TOKENS
    temperature: float = 0.0
    top_k: int = DEFAULT_TOP_K
    seed: int = DEFAULT_SEED
    eos_token_id: Optional[int] = None     # not in the reference's runtime: stop when sampled

    @property
    def is_greedy(self) -> bool:
        return not (self.temperature > 0.0)

    def effective_top_k(self, vocab: int) -> int:
        return max(1, min(int(self.top_k), vocab))

    def validate(self, vocab: int, max_device_top_k: Optional[int] = None) -> None:
        """`sampling.rs:301-317`, plus what this engine's kernel holds."""
        if isinstance(self.temperature, float) and math.isnan(self.temperature):
            raise ValueError("temperature must be a number")
        if self.temperature > 100.0:
            raise ValueError(f"temperature {self.temperature} is out of range (max 100)")
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if not 0 <= self.seed < (1 << 64):
            raise ValueError("seed must fit in 64 bits")
        if (not self.is_greedy and max_device_top_k is not None
                and self.effective_top_k(vocab) > max_device_top_k):
            raise ValueError(f"top_k {self.effective_top_k(vocab)} exceeds the {max_device_top_k} "
                             f"candidates the sampling kernel holds")
