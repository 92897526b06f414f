"""Per-request sampling options, with the reference's names and defaults
(include/inferx/scheduler/scheduler.h:19-65).  Greedy, temperature, top-k, top-p,
min-p, stop tokens, ``ignore_eos`` and the seed are honoured; penalties, minimum
tokens and log-probabilities are accepted only at their neutral values."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass
class SamplingParams:
    max_tokens: int = 16
    stop_tokens: Tuple[int, ...] = ()
    temperature: float = 0.0      # zero or below is greedy
    top_p: float = 1.0            # at or above 1 disables
    top_k: int = 0                # 0 disables
    min_p: float = 0.0            # 0 disables
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    min_tokens: int = 0
    ignore_eos: bool = False
    want_logprobs: bool = False
    top_logprobs: int = 0
    seed: int = 0

    def __post_init__(self):
        self.stop_tokens = tuple(int(t) for t in self.stop_tokens)
        if (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.repetition_penalty != 1.0 or self.min_tokens != 0
                or self.want_logprobs or self.top_logprobs):
            raise NotImplementedError(
                "penalties, min_tokens and logprobs are not part of this engine; "
                "leave them at their neutral values")
        if self.top_k < 0 or self.min_p < 0 or self.top_p <= 0:
            raise ValueError("top_k and min_p must not be negative and top_p must be positive")
