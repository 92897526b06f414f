"""Per-request sampling options, with the reference's names and defaults
(include/inferx/scheduler/scheduler.h:19-65).  Greedy, temperature, top-k, top-p,
min-p, stop tokens, ``ignore_eos`` and the seed; presence, frequency and repetition
penalties over the tokens generated so far; ``min_tokens`` (stop tokens cannot be chosen
before that many were generated); log-probabilities of the chosen token and of up to 20
alternatives."""
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
    presence_penalty: float = 0.0     # subtracted from every token generated so far
    frequency_penalty: float = 0.0    # ... times how often it was generated
    repetition_penalty: float = 1.0   # divides their positive logits, multiplies the others
    min_tokens: int = 0           # stop tokens are masked until this many were generated
    ignore_eos: bool = False
    want_logprobs: bool = False   # report the chosen token's log-probability
    top_logprobs: int = 0         # ... and this many most probable alternatives (20 at most)
    seed: int = 0

    def __post_init__(self):
        self.stop_tokens = tuple(int(t) for t in self.stop_tokens)
        if not self.repetition_penalty > 0.0:
            raise ValueError("repetition_penalty must be positive (1 turns it off)")
        if self.min_tokens < 0 or self.top_logprobs < 0:
            raise ValueError("min_tokens and top_logprobs must not be negative")
        if self.top_k < 0 or self.min_p < 0 or self.top_p <= 0:
            raise ValueError("top_k and min_p must not be negative and top_p must be positive")
