"""The engine: a model folder in, generated tokens out.

``Engine.create(EngineConfig)`` loads the model, sizes the cache, and builds the
scheduler, the executor and the sampler; ``generate`` runs requests to completion
through the prepare -> step -> sample -> commit loop of the reference's engine
thread (src/engine/engine.cc:526-666), here driven synchronously by the caller.
Option names and meanings are the reference's (src/support/options.cc:47-174;
``SchedulerConfig``, include/inferx/scheduler/scheduler.h:129-154); the cache is
sized as in src/engine/kv_autosize.cc:10-47: an explicit number of blocks, else an
explicit number of bytes, else ``utilization * total - used - 1 GiB``, and never
less than one sequence of ``max_model_len``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, Iterator, List, Mapping, Optional, Sequence

import torch

from ..cache.manager import is_paged_need, groups_for
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import RandomSource
from .executor import StepEntry
from .runtime import Runtime, load_model, parse_dtype
from .scheduler import Completion, Scheduler, SchedulerConfig, TokenDelta, TokenLogprob


@dataclass
class EngineConfig:
    model: Optional[str] = None            # folder with config.json and safetensors
    dtype: str = "bfloat16"                # bfloat16 | float32
    max_num_seqs: int = 8                  # sequences resident at once
    max_model_len: int = 2048              # prompt plus generation
    max_num_batched_tokens: int = 0        # tokens per step; 0 = max(2048, max_model_len)
    block_size: int = 16                   # tokens per cache page
    num_gpu_blocks_override: int = 0       # pages per cache group, if > 0
    kv_cache_memory_bytes: int = 0         # else bytes for the cache, if > 0
    gpu_memory_utilization: float = 0.92   # else this share of the device
    prefill_chunk: int = 0                 # per-prompt tokens per step; 0 = the budget only
    enforce_eager: bool = False            # no CUDA graphs for decode steps
    device: str = "cuda"
    # random weights instead of a folder: the config and a seed
    config_json: Optional[Mapping[str, Any]] = None
    seed: int = 0

    def batched_tokens(self) -> int:
        return self.max_num_batched_tokens or max(2048, self.max_model_len)


@dataclass
class Request:
    prompt_ids: Sequence[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    id: Optional[Hashable] = None


def cache_bytes_per_page(model, page_size: int) -> List[int]:
    """Bytes one page costs in each cache group (every entry of every layer of the
    group)."""
    needs = model.cache_needs()
    groups = groups_for(needs)
    out = []
    for g in groups:
        b = 0
        for layer in g.layers:
            for need in needs[layer]:
                if is_paged_need(need) and int(need.window) == g.window:
                    b += need.bytes_per_token(model.ctx.dtype) * page_size
        out.append(b)
    return out


def graph_reserve_bytes(cfg: EngineConfig, model) -> int:
    """Device memory to leave for recorded steps: each kept graph holds the logits of its
    wanted rows (at most one row per resident sequence, fp32 over the vocabulary), and
    all of them share one pool of activations sized by the largest step (some dozens of
    bytes per token and unit of width, taken generously)."""
    from .executor import GraphCache
    limits = GraphCache().limits
    spec = model.spec
    logits = (limits[True] + limits[False]) * cfg.max_num_seqs * spec.vocab_size * 4
    activations = cfg.batched_tokens() * spec.hidden * 64
    return logits + activations


def autosize_pages(cfg: EngineConfig, model, device) -> int:
    """Pages per cache group (src/engine/kv_autosize.cc:10-47)."""
    per_page = sum(cache_bytes_per_page(model, cfg.block_size)) or 1
    floor = -(-cfg.max_model_len // cfg.block_size)
    if cfg.num_gpu_blocks_override > 0:
        return cfg.num_gpu_blocks_override
    if cfg.kv_cache_memory_bytes > 0:
        return max(floor, cfg.kv_cache_memory_bytes // per_page)
    if torch.device(device).type != "cuda":
        return max(floor, cfg.max_num_seqs * floor)
    free, total = torch.cuda.mem_get_info(device)
    used = total - free
    budget = int(cfg.gpu_memory_utilization * total) - used - (1 << 30)
    if not cfg.enforce_eager:
        budget -= graph_reserve_bytes(cfg, model)
    # no more than every resident sequence at full length can use
    want = cfg.max_num_seqs * floor
    return max(floor, min(want, budget // per_page))


class Engine:
    def __init__(self, config: EngineConfig, model_config, runtime: Runtime, ops):
        self.config = config
        self.model_config = model_config
        self.runtime = runtime
        self.scheduler = Scheduler(
            SchedulerConfig(max_running=config.max_num_seqs,
                            max_batch_tokens=config.batched_tokens(),
                            max_seq_len=config.max_model_len,
                            max_prefill_chunk=config.prefill_chunk),
            runtime.manager)
        self.sampler = Sampler(ops, runtime.executor.device)
        self._next_id = 0
        self.tokens_generated = 0
        self.tokens_prefilled = 0
        # wall-clock seconds of the host's part of every step, by what it was spent on
        # (the reference reports the same split, docs/ARCHITECTURE.md:172-180): planning,
        # building and launching the step, waiting for the sampled ids, committing
        self.seconds = {"plan": 0.0, "launch": 0.0, "wait": 0.0, "commit": 0.0}

    # ------------------------------------------------------------------
    @classmethod
    def create(cls, config: EngineConfig, ops=None) -> "Engine":
        parse_dtype(config.dtype)
        if config.model is not None:
            mcfg, model = load_model(config.model, dtype=config.dtype, device=config.device,
                                     ops=ops)
        elif config.config_json is not None:
            mcfg, model = load_model(dtype=config.dtype, device=config.device,
                                     config_json=config.config_json,
                                     source=RandomSource(config.seed, device=config.device),
                                     ops=ops)
        else:
            raise ValueError("EngineConfig needs a model folder, or a config for random weights")
        pages = autosize_pages(config, model, config.device)
        runtime = Runtime(model, page_size=config.block_size, num_pages=pages,
                          max_slots=config.max_num_seqs,
                          use_graphs=not config.enforce_eager)
        return cls(config, mcfg, runtime, model.ctx.ops)

    # ------------------------------------------------------------------
    def submit(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None,
               request_id: Optional[Hashable] = None) -> Hashable:
        """Queue a request; returns its id.  The model's end-of-sequence ids join the
        stop tokens unless ``ignore_eos`` (src/engine/engine.cc:821-823)."""
        params = params or SamplingParams()
        if len(prompt_ids) >= self.config.max_model_len:
            raise ValueError(f"prompt of {len(prompt_ids)} tokens does not fit max_model_len "
                             f"{self.config.max_model_len}")
        vocab = self.runtime.vocab_size
        for t in prompt_ids:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        eos = tuple(getattr(self.model_config, "eos_token_ids", ()) or ())
        if eos and not params.ignore_eos:
            import dataclasses
            params = dataclasses.replace(
                params, stop_tokens=tuple(params.stop_tokens) + tuple(
                    t for t in eos if t not in params.stop_tokens))
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        self.scheduler.add_request(request_id, prompt_ids, params)
        return request_id

    def step(self) -> List[TokenDelta]:
        """One scheduler step; the tokens it produced."""
        clock = time.perf_counter
        t0 = clock()
        planned = self.scheduler.prepare_step()
        if not planned:
            return []
        entries = [StepEntry(e.id, e.tokens, [len(e.tokens) - 1] if e.sample else [])
                   for e in planned]
        t1 = clock()
        logits = self.runtime.executor.step(entries)
        sampled: List[int] = []
        rows = [e for e in planned if e.sample]
        ids = self.sampler(logits, rows) if rows else None
        lps = self.sampler.logprobs(logits, ids, rows) if rows else None
        t2 = clock()
        if ids is not None:
            sampled = ids.tolist()          # the one wait of the step
        records = self._logprob_records(sampled, lps) if lps is not None else None
        t3 = clock()
        deltas = self.scheduler.commit_step(sampled, records)
        t4 = clock()
        sec = self.seconds
        sec["plan"] += t1 - t0
        sec["launch"] += t2 - t1
        sec["wait"] += t3 - t2
        sec["commit"] += t4 - t3
        self.tokens_generated += len(sampled)
        self.tokens_prefilled += sum(len(e.tokens) for e in planned) - len(rows)
        return deltas

    @staticmethod
    def _logprob_records(sampled, lps):
        chosen_lp, top_ids, top_lps, ks = lps
        chosen_lp = chosen_lp.tolist()
        top_ids = top_ids.tolist() if top_ids is not None else None
        top_lps = top_lps.tolist() if top_lps is not None else None
        out = []
        for i, k in enumerate(ks):
            if k < 0:
                out.append(None)
                continue
            top = [(int(t), float(p)) for t, p in zip(top_ids[i][:k], top_lps[i][:k])
                   if t >= 0] if k > 0 else []
            out.append(TokenLogprob(int(sampled[i]), float(chosen_lp[i]), top))
        return out

    def stream(self) -> Iterator[TokenDelta]:
        """Run until nothing is left, yielding each token as it is produced."""
        while self.scheduler.has_work():
            for d in self.step():
                yield d

    def generate(self, requests: Sequence[Request]) -> List[Completion]:
        """Run the requests to completion; completions in the order of the requests."""
        ids = [self.submit(r.prompt_ids, r.params, r.id) for r in requests]
        done: Dict[Hashable, Completion] = {}
        while self.scheduler.has_work():
            self.step()
            for c in self.scheduler.take_completed():
                done[c.id] = c
        for c in self.scheduler.take_completed():
            done[c.id] = c
        self.runtime.executor.poll_errors()
        return [done[i] for i in ids]

    def stats(self) -> Dict[str, Any]:
        mgr = self.runtime.manager
        return {
            "steps": self.scheduler.steps,
            "preemptions": self.scheduler.preemptions,
            "tokens_generated": self.tokens_generated,
            "tokens_prefilled": self.tokens_prefilled,
            "graph_replays": self.runtime.executor.graph_replays,
            "graph_captures": self.runtime.executor.graph_captures,
            "capture_seconds": round(self.runtime.executor.capture_seconds, 4),
            "eager_steps": self.runtime.executor.eager_steps,
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "pages_free": [p.free_count for p in mgr.pools],
            "pages_total": [p.num_pages for p in mgr.pools],
            "cache_bytes": self.runtime.storage.bytes(),
            "host_seconds": {k: round(v, 4) for k, v in self.seconds.items()},
        }
