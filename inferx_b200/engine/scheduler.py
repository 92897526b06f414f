"""Continuous batching: admission, chunked prefill, decoding, finishing, preemption.

The scheduler holds all policy and touches no device: it produces lists of
(request, tokens, wanted place) for the step function and consumes sampled token
ids, exactly the split of the reference (include/inferx/scheduler/scheduler.h:
179-279).  Behaviour follows src/scheduler/scheduler.cc:

* admission (``Admit``, 294-370): first come first served while fewer than
  ``max_running`` run; a request longer than ``max_seq_len`` is retired at once;
  pages for the request's whole current token list (prompt plus anything generated
  before a preemption) are reserved at admission; if they cannot be had the
  request gives everything back and stays at the head of the queue.  Admission
  never preempts.
* token budget (``Plan``, 255-291): every step hands out ``max_batch_tokens``:
  sequences with exactly one token pending (decodes, and the last token of a
  prompt) first, then prompts first come first served, each taking what is left of
  the budget (chunked prefill).  ``max_prefill_chunk`` additionally caps what one
  prompt takes in one step (the reference has only the budget).
* when pages run out while growing (``PrepareStep``, 455-510): the most recently
  admitted sequence is preempted, or the next-newest when the needy one is the
  newest; a sequence running alone is retired with ``out_of_memory``; then the plan
  is made again.  Preemption is by recompute (``Preempt``, 206-229): pages freed,
  tokens kept (prompt and generated), back to the *front* of the queue; when
  admitted again it prefills all of them and goes on.
* a sequence that has filled ``max_seq_len`` is retired with ``context_limit``.
* commit (``CommitStep``, 677-758): sampled tokens are appended; a stop token
  finishes with ``stop_token``, ``max_tokens`` generated with ``max_tokens``.
* seeds: the row's seed is ``seed ^ (0x9e3779b97f4a7c15 * len(tokens))``
  (scheduler.cc:613-615), so a draw depends on the position, not on the batch.
* penalties (scheduler.cc:617-645): a row whose request has a penalty carries the distinct
  tokens it has generated with their counts, most recent first, at most 256 of them (the
  counts cover the whole generation also when the set is cut).  ``min_tokens``
  (647-657): while fewer have been generated the row carries its stop tokens (16 at most)
  to be masked.  Log-probabilities (659-664): -1 when not wanted, else how many
  alternatives (20 at most); ``commit_step`` attaches them to the tokens.
"""
from __future__ import annotations

import collections
from dataclasses import dataclass
from typing import Deque, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

STOP_TOKEN = "stop_token"
MAX_TOKENS = "max_tokens"
CANCELLED = "cancelled"
OUT_OF_MEMORY = "out_of_memory"
CONTEXT_LIMIT = "context_limit"

_MASK64 = (1 << 64) - 1


@dataclass
class SchedulerConfig:
    max_running: int = 8            # sequences resident at once (--max-num-seqs)
    max_batch_tokens: int = 2048    # tokens per step over the batch (--max-num-batched-tokens)
    max_seq_len: int = 2048         # prompt plus generation (--max-model-len)
    max_prefill_chunk: int = 0      # per-prompt cap per step; 0 = the budget only


PENALTY_HISTORY_CAP = 256       # distinct generated tokens a row's penalties look at
MASK_CAP = 16                   # stop tokens masked under min_tokens
MAX_TOP_LOGPROBS = 20


@dataclass
class TokenLogprob:
    """Of one generated token: its log-probability and the most probable alternatives
    (token id, log-probability), most probable first."""
    token: int
    logprob: float
    top: List[Tuple[int, float]]


@dataclass
class Completion:
    id: Hashable
    output_tokens: List[int]
    reason: str
    logprobs: Optional[List[TokenLogprob]] = None     # when the request asked for them


@dataclass
class TokenDelta:
    id: Hashable
    token: int
    finish: Optional[str] = None
    logprob: Optional[TokenLogprob] = None


@dataclass
class PlannedEntry:
    id: Hashable
    tokens: List[int]
    sample: bool                 # the portion reaches the end of the tokens: sample after it
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int = 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    history: Tuple[Tuple[int, int], ...] = ()   # (token, count) generated so far, newest first
    masked: Tuple[int, ...] = ()                # tokens that must not be chosen in this step
    logprobs_k: int = -1                        # -1: none; else how many alternatives


@dataclass
class _Sequence:
    id: Hashable
    tokens: List[int]
    prompt_len: int
    params: SamplingParams
    cached: int = 0
    cancelled: bool = False
    logprobs: Optional[List[TokenLogprob]] = None

    def pending(self) -> int:
        return len(self.tokens) - self.cached

    def generated(self) -> int:
        return len(self.tokens) - self.prompt_len


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager):
        if config.max_running <= 0 or config.max_batch_tokens <= 0 or config.max_seq_len <= 0:
            raise ValueError("scheduler config has a non-positive bound")
        self.config = config
        self.cache = cache
        self.waiting: Deque[_Sequence] = collections.deque()
        self.running: List[_Sequence] = []
        self.completed: List[Completion] = []
        self.preemptions = 0
        self.steps = 0
        self._planned: List[PlannedEntry] = []
        self._planned_seqs: List[_Sequence] = []
        self._ids = set()

    # -- requests --------------------------------------------------------------
    def add_request(self, rid: Hashable, prompt: Sequence[int], params: SamplingParams) -> None:
        if len(prompt) == 0:
            raise ValueError("a request needs a non-empty prompt")
        if params.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if rid in self._ids:
            raise ValueError(f"request id {rid!r} is already in use")
        self._ids.add(rid)
        self.waiting.append(_Sequence(rid, [int(t) for t in prompt], len(prompt), params))

    def cancel(self, rid: Hashable) -> None:
        """Takes effect at the next ``prepare_step``."""
        for seq in list(self.waiting) + self.running:
            if seq.id == rid:
                seq.cancelled = True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def take_completed(self) -> List[Completion]:
        out, self.completed = self.completed, []
        return out

    # -- internals -------------------------------------------------------------
    def _retire(self, seq: _Sequence, reason: str) -> None:
        self.completed.append(Completion(seq.id, seq.tokens[seq.prompt_len:], reason,
                                         seq.logprobs))
        if self.cache.has(seq.id):
            self.cache.close(seq.id)
        self._ids.discard(seq.id)

    def _preempt(self, index: int) -> None:
        victim = self.running.pop(index)
        self.cache.close(victim.id)
        victim.cached = 0
        self.waiting.appendleft(victim)
        self.preemptions += 1

    def _admit(self) -> None:
        cfg = self.config
        while self.waiting and len(self.running) < cfg.max_running:
            seq = self.waiting[0]
            if seq.cancelled:
                self.waiting.popleft()
                self._retire(seq, CANCELLED)
                continue
            needed = len(seq.tokens)
            if needed > cfg.max_seq_len:
                self.waiting.popleft()
                self._retire(seq, OUT_OF_MEMORY)
                continue
            if self.cache.open(seq.id) is None:
                return                      # no state slot free: stay queued
            if not self.cache.reserve(seq.id, needed):
                self.cache.close(seq.id)    # give everything back, stay first in line
                return
            seq.cached = 0
            self.waiting.popleft()
            self.running.append(seq)

    def _plan(self) -> List[int]:
        cfg = self.config
        take = [0] * len(self.running)
        budget = cfg.max_batch_tokens
        for s, seq in enumerate(self.running):
            if budget <= 0:
                break
            if seq.pending() == 1:
                take[s] = 1
                budget -= 1
        for s, seq in enumerate(self.running):
            if budget <= 0:
                break
            pending = seq.pending()
            if pending <= 1:
                continue
            chunk = min(pending, budget)
            if cfg.max_prefill_chunk > 0:
                chunk = min(chunk, cfg.max_prefill_chunk)
            take[s] = chunk
            budget -= chunk
        return take

    # -- the step ----------------------------------------------------------------
    def prepare_step(self) -> List[PlannedEntry]:
        """Decide the next batch; pages for it are reserved when this returns.
        An empty list means there is nothing to run."""
        for seq in [s for s in self.running if s.cancelled]:
            self.running.remove(seq)
            self._retire(seq, CANCELLED)
        self._admit()
        while not self.running and self.waiting:
            # nothing runs, so the cache is empty, and still the head of the queue
            # could not be admitted: it can never fit
            self._retire(self.waiting.popleft(), OUT_OF_MEMORY)
            self._admit()
        take: List[int] = []
        initial = len(self.running)
        for _attempt in range(initial + 1):
            if not self.running:
                break
            take = self._plan()
            replan = False
            for s, seq in enumerate(self.running):
                if take[s] == 0:
                    continue
                target = seq.cached + take[s]
                if target > self.config.max_seq_len:
                    self.running.pop(s)
                    self._retire(seq, CONTEXT_LIMIT)
                    replan = True
                    break
                if self.cache.reserve(seq.id, target):
                    continue
                victim = len(self.running) - 1
                if victim == s:
                    if len(self.running) == 1:
                        self.running.pop(s)
                        self._retire(seq, OUT_OF_MEMORY)
                        replan = True
                        break
                    victim = len(self.running) - 2
                self._preempt(victim)
                replan = True
                break
            if not replan:
                break
        self._planned, self._planned_seqs = [], []
        if not self.running:
            return []
        for s, seq in enumerate(self.running):
            n = take[s] if s < len(take) else 0
            if n == 0:
                continue
            last = seq.cached + n == len(seq.tokens)
            p = seq.params
            entry = PlannedEntry(
                id=seq.id, tokens=seq.tokens[seq.cached:seq.cached + n], sample=last,
                temperature=p.temperature, top_p=p.top_p, top_k=p.top_k, min_p=p.min_p,
                seed=(p.seed ^ ((0x9E3779B97F4A7C15 * len(seq.tokens)) & _MASK64)) & _MASK64)
            if last:
                self._sampling_extras(entry, seq)
            self._planned.append(entry)
            self._planned_seqs.append(seq)
        self.steps += 1
        return self._planned

    @staticmethod
    def _sampling_extras(entry: PlannedEntry, seq: _Sequence) -> None:
        p = seq.params
        if (p.presence_penalty != 0.0 or p.frequency_penalty != 0.0
                or p.repetition_penalty != 1.0) and seq.generated() > 0:
            entry.presence_penalty = p.presence_penalty
            entry.frequency_penalty = p.frequency_penalty
            entry.repetition_penalty = p.repetition_penalty
            counts = collections.Counter(seq.tokens[seq.prompt_len:])
            newest_first = []
            for tok in reversed(seq.tokens[seq.prompt_len:]):
                if tok in counts and len(newest_first) < PENALTY_HISTORY_CAP:
                    newest_first.append((tok, counts.pop(tok)))
            entry.history = tuple(newest_first)
        if seq.generated() < p.min_tokens:
            entry.masked = tuple(p.stop_tokens[:MASK_CAP])
        if p.want_logprobs:
            entry.logprobs_k = min(int(p.top_logprobs), MAX_TOP_LOGPROBS)

    def commit_step(self, sampled: Sequence[int],
                    logprobs: Optional[Sequence[Optional[TokenLogprob]]] = None
                    ) -> List[TokenDelta]:
        """Record that the planned batch ran; ``sampled`` holds one token per entry
        that asked for a sample, in entry order, and ``logprobs`` (when given) what goes
        with each of them, None for rows that did not ask."""
        want = sum(1 for e in self._planned if e.sample)
        if len(sampled) != want:
            raise ValueError(f"{len(sampled)} sampled tokens for {want} rows that asked")
        if logprobs is not None and len(logprobs) != want:
            raise ValueError(f"{len(logprobs)} log-probability records for {want} rows")
        lp_it = iter(logprobs) if logprobs is not None else None
        deltas: List[TokenDelta] = []
        finished = []
        it = iter(sampled)
        for entry, seq in zip(self._planned, self._planned_seqs):
            n = len(entry.tokens)
            self.cache.advance(seq.id, n)
            seq.cached += n
            if not entry.sample:
                continue
            tok = int(next(it))
            seq.tokens.append(tok)
            lp = next(lp_it) if lp_it is not None else None
            if lp is not None:
                if seq.logprobs is None:
                    seq.logprobs = []
                # after a preemption the tokens are kept and so are their records
                seq.logprobs.append(lp)
            reason = None
            if tok in seq.params.stop_tokens:
                reason = STOP_TOKEN
            elif seq.generated() >= seq.params.max_tokens:
                reason = MAX_TOKENS
            deltas.append(TokenDelta(seq.id, tok, reason, lp))
            if reason:
                finished.append((seq, reason))
        for seq, reason in finished:
            self.running.remove(seq)
            self._retire(seq, reason)
        self._planned, self._planned_seqs = [], []
        return deltas
