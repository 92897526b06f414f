"""The step function: one batch of (request, its next tokens) through the model.

The executor holds all the device work and no policy (the reference's split,
README.md:46-49, docs/ARCHITECTURE.md:101).  ``step`` takes, for each request in
the batch, the tokens to run now (a portion of a prompt, or one decoded token)
and the places among them whose logits are wanted; it runs exactly those tokens
as one batch against the cache earlier steps left and returns the fp32 logits
``[wanted, vocab]`` in the order of the entries.  It corresponds to the
reference's ``Qwen2Model::Step`` (src/model/qwen2.cc:2246-2277) with
``PrepareBatchInputs`` (qwen2.cc:564-817) and ``ForwardBatch::Validate``
(src/model/forward_batch.cc:5-93): rows grouped by sequence, contiguous
positions, every index array checked on the host before anything is launched.
All index arrays of a step travel in one pinned staging buffer and one copy.

Steps in which every request brings exactly one token can be replayed from a CUDA
graph captured per (batch size, block-table width), the reference's
``CaptureDecodeGraph`` / ``FindGraph(tokens, seqs, blocks)``
(qwen2.cc:1588-1712, 2210-2218); like the reference the choice is by shape only.

The executor reads the cache manager (lengths, block tables, slots) and never
changes it, except for zeroing the state of slots newly handed out.  Pages must
have been reserved by the caller (the scheduler or the replay tool), which also
advances the request's length after the step.
"""
from __future__ import annotations

import time
import warnings
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..parts.base import GroupView, StepContext


class StepError(ValueError):
    """A batch the step function refuses before launching anything."""


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()   # indices into ``tokens`` whose logits are wanted


def _pad4(n: int) -> int:
    return (n + 3) & ~3


def _bucket(n: int) -> int:
    """Block-table widths a graph is captured for: powers of two from 8."""
    b = 8
    while b < n:
        b *= 2
    return b


# order of the index arrays inside a step's staging buffer
_TOKENS, _POSITIONS, _SEQ_OF_TOKEN, _CU_Q, _Q_POS0, _KV_LEN, _STATE_SLOT, _LOGIT_ROWS, \
    _CU_Q_PROMPT = range(9)
_FIXED_SEGS = 9        # then, per cache group: slots, block table


@dataclass
class _Layout:
    """Host-side description of one batch: every index array of the step laid out in one
    int32 buffer (``buf``), with the offset and length of each."""
    T: int
    S: int
    R: int
    buf: "np.ndarray"
    offs: List[int]
    lens: List[int]
    total: int
    widths: List[int]          # block-table width per group
    q_lens: List[int]
    kv_lens: List[int]
    wanted: Tuple[int, ...]
    num_decode: int = 0        # sequences with a single token; they come first
    state_slots: Tuple[int, ...] = ()
    first_live: Tuple[Tuple[int, ...], ...] = ()   # per group, per sequence


@dataclass
class _Graph:
    graph: "torch.cuda.CUDAGraph"
    dev: torch.Tensor
    hosts: List[torch.Tensor]          # two pinned staging buffers, used in turn
    copied: List[Optional["torch.cuda.Event"]]
    logits: Optional[torch.Tensor]
    turn: int = 0


class GraphCache:
    """Which step shapes are kept as recorded CUDA graphs, and for how long.

    A step's shape is: how many tokens each sequence brings (in batch order), the width
    of each group's block table (rounded up to a bucket) and the wanted rows.  Steps of
    single tokens are recorded the second time their shape is seen; other shapes (prompt
    portions, mixed batches) the third time: prompts rarely repeat a shape exactly,
    except for full portions of long prompts and for benchmarks.  Both kinds are kept
    least-recently-used up to a bound of their own, because every recorded step holds
    device memory (its index arrays, its logits, its share of the graph pool): a serving
    run whose batch sizes and contexts wander would otherwise keep one for every
    (batch size, table width) it ever met.  (The reference records a fixed list of decode
    shapes at start-up, src/model/qwen2.cc:1588-1712.)  Pure bookkeeping: it never
    touches a device."""

    def __init__(self, decode_graphs: int = 64, prompt_graphs: int = 4,
                 decode_seen: int = 2, prompt_seen: int = 3, seen_shapes: int = 4096):
        self.limits = {True: int(decode_graphs), False: int(prompt_graphs)}
        self.need_seen = {True: int(decode_seen), False: int(prompt_seen)}
        self.seen_shapes = int(seen_shapes)
        self._kept = {True: {}, False: {}}     # decode? -> {key: graph}; oldest first
        self._seen: Dict[Tuple, int] = {}
        self.evictions = 0

    def __len__(self) -> int:
        return len(self._kept[True]) + len(self._kept[False])

    def count(self, decode: bool) -> int:
        return len(self._kept[decode])

    def get(self, key):
        """The recorded step of this shape, marked most recently used; or None."""
        for kept in self._kept.values():
            if key in kept:
                kept[key] = kept.pop(key)      # dicts keep insertion order: last = newest
                return kept[key]
        return None

    def should_record(self, key, decode: bool) -> bool:
        """Count a sighting of a shape that is not kept; True when it is due."""
        if len(self._seen) >= self.seen_shapes:
            self._seen.clear()
        n = self._seen[key] = self._seen.get(key, 0) + 1
        return n >= self.need_seen[decode]

    def put(self, key, graph, decode: bool) -> None:
        kept = self._kept[decode]
        while len(kept) >= max(1, self.limits[decode]):
            del kept[next(iter(kept))]         # the least recently used goes
            self.evictions += 1
        kept[key] = graph
        self._seen.pop(key, None)


class Executor:
    def __init__(self, model, manager: CacheManager, storage: CacheStorage,
                 use_graphs: bool = False):
        self.model = model
        self.manager = manager
        self.storage = storage
        self.device = storage.device
        self.vocab = model.spec.vocab_size
        self.caches = storage.layer_caches(model.spec.schedule)
        self.steps_run = 0
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda"
        self._graphs = GraphCache()
        self._graph_pool = None
        self._capture_stream = None
        self.graph_replays = 0
        self.graph_captures = 0
        self.eager_steps = 0
        self.capture_seconds = 0.0        # host time spent recording steps
        self._staging: List[list] = []
        self._staging_turn = -1
        self.last_h2d_bytes = 0

    # ------------------------------------------------------------------
    def _layout(self, entries: Sequence[StepEntry], bucket_tables: bool) -> _Layout:
        """Validate the batch and lay its index arrays out in one int32 buffer."""
        mgr = self.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        n_groups = len(mgr.groups)
        ps = mgr.page_size
        vocab = self.vocab
        # single tokens first, prompt portions after them, each kind in the order given:
        # attention can then treat the two parts of a mixed batch as two plain batches
        order = sorted(range(len(entries)), key=lambda i: len(entries[i].tokens) != 1)
        S = len(entries)
        seen = set()
        starts: List[int] = []
        q_lens: List[int] = []
        for i in order:
            e = entries[i]
            rid = e.request
            if rid in seen:
                raise StepError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            if not mgr.has(rid):
                raise StepError(f"request {rid!r} has no cache (open it first)")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {rid!r} brings no tokens")
            start = mgr.length(rid)
            if start + n > mgr.capacity(rid):
                raise StepError(
                    f"request {rid!r}: positions {start}..{start + n - 1} exceed the "
                    f"{mgr.capacity(rid)} tokens its pages hold (reserve first)")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {rid!r}: wanted place {int(w)} is not among "
                                    f"its {n} tokens")
            starts.append(start)
            q_lens.append(n)
        T = sum(q_lens)
        R = sum(len(e.want) for e in entries)
        num_decode = sum(1 for n in q_lens if n == 1)
        tables = [[mgr.table(entries[i].request, g) for i in order] for g in range(n_groups)]
        widths = []
        for g in range(n_groups):
            mb = max(1, max(len(r) for r in tables[g]))
            widths.append(_bucket(mb) if bucket_tables else mb)
        lens = [T, T, T, S + 1, S, S, S, R, S - num_decode + 1]
        for g in range(n_groups):
            lens += [T, S * widths[g]]
        offs, total = [], 0
        for n in lens:
            offs.append(total)
            total += _pad4(n)
        total = max(total, 4)
        buf = np.zeros(total, dtype=np.int32)

        def seg(k):
            return buf[offs[k]:offs[k] + lens[k]]

        tok, pos, seq_of = seg(_TOKENS), seg(_POSITIONS), seg(_SEQ_OF_TOKEN)
        cu_q, q_pos0, kv_len, state_slot = seg(_CU_Q), seg(_Q_POS0), seg(_KV_LEN), seg(_STATE_SLOT)
        slot_segs = [seg(_FIXED_SEGS + 2 * g) for g in range(n_groups)]
        base_of = [0] * S
        base = 0
        for s, i in enumerate(order):
            e = entries[i]
            rid, n, start = e.request, q_lens[s], starts[s]
            base_of[i] = base
            if n == 1:
                t = int(e.tokens[0])
                if not (0 <= t < vocab):
                    raise StepError(f"request {rid!r}: token id {t} is outside the "
                                    f"vocabulary of {vocab}")
                tok[base] = t
                pos[base] = start
                seq_of[base] = s
                for g in range(n_groups):
                    page = tables[g][s][start // ps]
                    if page < 0:
                        raise StepError(f"request {rid!r}: the page of position {start} was "
                                        "given back")
                    slot_segs[g][base] = page * ps + start % ps
            else:
                ids = np.asarray(e.tokens, dtype=np.int64)
                if ids.min() < 0 or ids.max() >= vocab:
                    bad = int(ids[(ids < 0) | (ids >= vocab)][0])
                    raise StepError(f"request {rid!r}: token id {bad} is outside the "
                                    f"vocabulary of {vocab}")
                tok[base:base + n] = ids
                p = np.arange(start, start + n, dtype=np.int64)
                pos[base:base + n] = p
                seq_of[base:base + n] = s
                for g in range(n_groups):
                    row = np.frombuffer(tables[g][s], dtype=np.int32)
                    pages = row[p // ps].astype(np.int64)
                    if pages.min() < 0:
                        gone = int(p[pages < 0][0])
                        raise StepError(f"request {rid!r}: the page of position {gone} was "
                                        "given back")
                    slot_segs[g][base:base + n] = pages * ps + p % ps
            cu_q[s + 1] = base + n
            q_pos0[s] = start
            kv_len[s] = start + n
            state_slot[s] = mgr.slot(rid)
            base += n
        wanted: List[int] = []
        for i, e in enumerate(entries):      # logits come back in the order of the entries
            wanted.extend(base_of[i] + int(w) for w in e.want)
        if R:
            seg(_LOGIT_ROWS)[:] = wanted
        seg(_CU_Q_PROMPT)[:] = cu_q[num_decode:] - cu_q[num_decode]
        for g in range(n_groups):
            mb = widths[g]
            view = seg(_FIXED_SEGS + 2 * g + 1).reshape(S, mb)
            view.fill(-1)
            for s, row in enumerate(tables[g]):
                if len(row):
                    view[s, :len(row)] = np.frombuffer(row, dtype=np.int32)
        return _Layout(T=T, S=S, R=R, buf=buf, offs=offs, lens=lens, total=total, widths=widths,
                       q_lens=q_lens, kv_lens=[a + n for a, n in zip(starts, q_lens)],
                       wanted=tuple(wanted), num_decode=num_decode,
                       state_slots=tuple(int(x) for x in state_slot),
                       first_live=tuple(tuple(mgr.first_live(entries[i].request, g)
                                              for i in order) for g in range(n_groups)))

    @staticmethod
    def _fill(host: torch.Tensor, lay: _Layout) -> None:
        host.numpy()[:lay.total] = lay.buf

    def _context(self, dev: torch.Tensor, lay: _Layout, static: bool):
        mgr = self.manager

        def seg(i):
            return dev[lay.offs[i]:lay.offs[i] + lay.lens[i]]

        groups = []
        for g, grp in enumerate(mgr.groups):
            groups.append(GroupView(
                block_table=seg(_FIXED_SEGS + 2 * g + 1).view(lay.S, lay.widths[g]),
                slots=seg(_FIXED_SEGS + 2 * g), page_size=mgr.page_size, window=grp.window,
                first_live=None if static else list(lay.first_live[g])))
        max_kv = max(lay.kv_lens)
        if static:   # a captured graph must hold for every length its table width allows
            max_kv = max(w for w in lay.widths) * mgr.page_size if lay.widths else max_kv
        ctx = StepContext(
            num_tokens=lay.T, num_seqs=lay.S, token_ids=seg(_TOKENS), positions=seg(_POSITIONS),
            seq_of_token=seg(_SEQ_OF_TOKEN), cu_q=seg(_CU_Q), q_pos0=seg(_Q_POS0),
            kv_len=seg(_KV_LEN), state_slot=seg(_STATE_SLOT),
            groups=groups, max_q_len=max(lay.q_lens), max_kv_len=max_kv,
            q_lens=list(lay.q_lens), kv_lens=None if static else list(lay.kv_lens),
            state_slots=None if static else list(lay.state_slots), captured=static,
            all_decode=all(n == 1 for n in lay.q_lens), num_decode_seqs=lay.num_decode,
            cu_q_prompt=seg(_CU_Q_PROMPT))
        return ctx, (seg(_LOGIT_ROWS) if lay.R else None)

    # Index arrays of steps that are not replayed travel through a small ring of pinned
    # staging buffers that are kept: page-locking host memory costs far more than a step's
    # copy, so it is not done per step.  A buffer is reused once the copy that last read it
    # has completed (an event recorded behind that copy).
    STAGING_BUFFERS = 4

    def _upload(self, lay: _Layout) -> torch.Tensor:
        """The step's index arrays on the device (one asynchronous copy)."""
        if self.device.type != "cuda":
            host = torch.zeros(lay.total, dtype=torch.int32)
            self._fill(host, lay)
            return host
        ring = self._staging
        i = self._staging_turn = (self._staging_turn + 1) % self.STAGING_BUFFERS
        if len(ring) <= i:
            ring.append([None, None])
        buf, ev = ring[i]
        if ev is not None:
            ev.synchronize()
        if buf is None or buf.numel() < lay.total:
            buf = torch.zeros(max(lay.total, 4096), dtype=torch.int32).pin_memory()
        self._fill(buf, lay)
        dev = torch.empty(lay.total, dtype=torch.int32, device=self.device)
        dev.copy_(buf[:lay.total], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        ring[i] = [buf, ev]
        return dev

    def build_context(self, entries: Sequence[StepEntry]):
        """(StepContext, logit_rows tensor or None, number of wanted rows) for an eager step."""
        lay = self._layout(entries, bucket_tables=False)
        dev = self._upload(lay)
        self.last_h2d_bytes = lay.total * 4
        ctx, rows = self._context(dev, lay, static=False)
        return ctx, rows, lay.R

    # ------------------------------------------------------------------
    def _graph_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        lay = self._layout(entries, bucket_tables=True)
        decode = lay.num_decode == lay.S
        key = (lay.S if decode else tuple(lay.q_lens), tuple(lay.widths), lay.wanted)
        slot = self._graphs.get(key)
        if slot is None and not self._graphs.should_record(key, decode):
            # The first step of a shape runs eagerly: kernels are loaded, attributes
            # set and the library's plans made outside of any capture.  It is built like
            # a recorded step (bucketed tables, no per-step host values), so that a part
            # which cannot be recorded fails here, at the first step, and not later.
            dev = self._upload(lay)
            self.last_h2d_bytes = lay.total * 4
            ctx, rows = self._context(dev, lay, static=True)
            self.eager_steps += 1
            return self.model.forward(ctx, self.caches, rows)
        if slot is None:
            t_capture = time.perf_counter()
            host = torch.zeros(lay.total, dtype=torch.int32).pin_memory()
            dev = torch.zeros(lay.total, dtype=torch.int32, device=self.device)
            self._fill(host, lay)
            dev.copy_(host, non_blocking=True)
            ctx, rows = self._context(dev, lay, static=True)
            torch.cuda.current_stream(self.device).synchronize()
            if self._graph_pool is None or len(self._graphs) == 0:
                # a pool lives as long as a graph recorded into it: with none left, the
                # old handle names nothing
                self._graph_pool = torch.cuda.graph_pool_handle()
            graph = torch.cuda.CUDAGraph()
            # One memory pool for all recorded steps: they run one after the other, so
            # their activations can live in the same memory; a step's logits stay
            # allocated while its graph is kept and are not handed to a later recording.
            logits = self._record(graph, lambda: self.model.forward(ctx, self.caches, rows))
            slot = _Graph(graph, dev, [host, torch.zeros_like(host).pin_memory()], [None, None],
                          logits)
            self._graphs.put(key, slot, decode)
            self.graph_captures += 1
            self.capture_seconds += time.perf_counter() - t_capture
        else:
            i = slot.turn = 1 - slot.turn
            if slot.copied[i] is not None:
                slot.copied[i].synchronize()   # the copy that last read this buffer is done
            self._fill(slot.hosts[i], lay)
            slot.dev.copy_(slot.hosts[i], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            slot.copied[i] = ev
        self.last_h2d_bytes = lay.total * 4
        slot.graph.replay()
        self.graph_replays += 1
        return slot.logits

    def _record(self, graph, run):
        """Record ``run()`` into ``graph`` on a stream of its own.  This is what
        ``torch.cuda.graph`` does, without the garbage collection and the emptying of the
        allocator's cache that it starts with: a serving run records a few dozen step
        shapes while it runs, and those two cost more than the recording itself (and the
        emptied cache makes the next eager steps allocate from the driver again)."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        side, main = self._capture_stream, torch.cuda.current_stream(self.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            graph.capture_begin(pool=self._graph_pool)
            try:
                out = run()
            except BaseException:
                try:                 # leave capture mode, then report what went wrong
                    with warnings.catch_warnings():
                        warnings.simplefilter("ignore")      # "the graph is empty"
                        graph.capture_end()
                except Exception:
                    pass
                raise
            graph.capture_end()
        main.wait_stream(side)
        return out

    # ------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the batch; fp32 logits ``[wanted, vocab]`` on the device, or None.

        With graphs on, the logits of a replayed step live in the graph's own
        buffer and are overwritten by the next step of the same shape."""
        fresh = self.manager.take_fresh_slots()
        if fresh:
            self.storage.zero_slots(fresh)
        self.steps_run += 1
        if self.steps_run % self.ERROR_POLL_STEPS == 0:
            self.poll_errors()
        if self.use_graphs:
            return self._graph_step(entries)
        ctx, rows, _ = self.build_context(entries)
        self.eager_steps += 1
        return self.model.forward(ctx, self.caches, rows)

    # Kernels with bounded waits record a wait that ran out in a status word on the
    # device instead of hanging; reading it synchronises, so it is read now and then
    # (and by whoever ends a run) rather than every step.
    ERROR_POLL_STEPS = 64

    def poll_errors(self) -> None:
        ops = getattr(getattr(self.model, "ctx", None), "ops", None)
        check = getattr(ops, "check_async_errors", None)
        if check is not None:
            check()
