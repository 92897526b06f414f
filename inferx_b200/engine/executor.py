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

The executor reads the cache manager (lengths, block tables, slots) and never
changes it, except for zeroing the state of slots newly handed out.  Pages must
have been reserved by the caller (the scheduler or the replay tool), which also
advances the request's length after the step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

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


class Executor:
    def __init__(self, model, manager: CacheManager, storage: CacheStorage):
        self.model = model
        self.manager = manager
        self.storage = storage
        self.device = storage.device
        self.vocab = model.spec.vocab_size
        self.caches = storage.layer_caches(model.spec.schedule)
        self.steps_run = 0

    # ------------------------------------------------------------------
    def build_context(self, entries: Sequence[StepEntry]):
        """Validate the batch and lay its index arrays out for the device.

        Returns (StepContext, logit_rows tensor or None, number of wanted rows)."""
        mgr = self.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        token_ids: List[int] = []
        positions: List[int] = []
        seq_of_token: List[int] = []
        cu_q = [0]
        q_pos0: List[int] = []
        kv_len: List[int] = []
        state_slot: List[int] = []
        logit_rows: List[int] = []
        slots = [[] for _ in mgr.groups]
        ps = mgr.page_size
        for s, e in enumerate(entries):
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if not mgr.has(e.request):
                raise StepError(f"request {e.request!r} has no cache (open it first)")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            start = mgr.length(e.request)
            if start + n > mgr.capacity(e.request):
                raise StepError(
                    f"request {e.request!r}: positions {start}..{start + n - 1} exceed the "
                    f"{mgr.capacity(e.request)} tokens its pages hold (reserve first)")
            for tok in e.tokens:
                if not (0 <= int(tok) < self.vocab):
                    raise StepError(f"request {e.request!r}: token id {tok} is outside the "
                                    f"vocabulary of {self.vocab}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.request!r}: wanted place {w} is not among "
                                    f"its {n} tokens")
                logit_rows.append(len(token_ids) + int(w))
            for g in range(len(mgr.groups)):
                table = mgr.table(e.request, g)
                for p in range(start, start + n):
                    page = table[p // ps]
                    if page < 0:
                        raise StepError(f"request {e.request!r}: page of position {p} was "
                                        "given back")
                    slots[g].append(page * ps + p % ps)
            token_ids += [int(t) for t in e.tokens]
            positions += list(range(start, start + n))
            seq_of_token += [s] * n
            cu_q.append(cu_q[-1] + n)
            q_pos0.append(start)
            kv_len.append(start + n)
            state_slot.append(mgr.slot(e.request))
        T, S, R = len(token_ids), len(entries), len(logit_rows)
        max_blocks = []
        tables = []
        for g in range(len(mgr.groups)):
            rows = [mgr.table(e.request, g) for e in entries]
            mb = max(1, max(len(r) for r in rows))
            flat: List[int] = []
            for r in rows:
                flat += r + [-1] * (mb - len(r))
            max_blocks.append(mb)
            tables.append(flat)

        # one pinned staging buffer, one copy
        segs = [token_ids, positions, seq_of_token, cu_q, q_pos0, kv_len, state_slot, logit_rows]
        for g in range(len(mgr.groups)):
            segs += [slots[g], tables[g]]
        offs, total = [], 0
        for sgm in segs:
            offs.append(total)
            total += _pad4(len(sgm))
        host = torch.zeros(max(total, 4), dtype=torch.int32)
        for o, sgm in zip(offs, segs):
            if sgm:
                host[o:o + len(sgm)] = torch.tensor(sgm, dtype=torch.int32)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)

        def seg(i):
            return dev[offs[i]:offs[i] + len(segs[i])]

        groups = []
        for g, grp in enumerate(mgr.groups):
            groups.append(GroupView(block_table=seg(9 + 2 * g).view(S, max_blocks[g]),
                                    slots=seg(8 + 2 * g), page_size=ps, window=grp.window))
        q_lens = [cu_q[i + 1] - cu_q[i] for i in range(S)]
        ctx = StepContext(
            num_tokens=T, num_seqs=S, token_ids=seg(0), positions=seg(1), seq_of_token=seg(2),
            cu_q=seg(3), q_pos0=seg(4), kv_len=seg(5), state_slot=seg(6), groups=groups,
            max_q_len=max(q_lens), max_kv_len=max(kv_len), q_lens=q_lens, kv_lens=list(kv_len),
            all_decode=all(n == 1 for n in q_lens))
        return ctx, (seg(7) if R else None), R

    # ------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the batch; fp32 logits ``[wanted, vocab]`` on the device, or None."""
        fresh = self.manager.take_fresh_slots()
        if fresh:
            self.storage.zero_slots(fresh)
        ctx, rows, R = self.build_context(entries)
        logits = self.model.forward(ctx, self.caches, rows)
        self.steps_run += 1
        return logits
