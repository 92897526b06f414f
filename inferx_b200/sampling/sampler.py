"""Turns a step's logits into token ids on the device.

One kernel launch per step for all rows: greedy rows (temperature <= 0) take the
argmax with ties to the lower index (src/backends/cuda/ops/layers.cu:413-452); the
others draw from softmax(logits / t) restricted by top-k, min-p and top-p with one
uniform keyed by the row's seed (layers.cu:1051-1303).  A batch that is all greedy
skips the parameter upload.

Before that, rows whose request has a penalty or is under its ``min_tokens`` get their
logits changed in place (one more launch, only in steps that have such a row:
layers.cu:1310-1347, src/engine/host_sampling.cc:21-48); after it, rows that want
log-probabilities get them computed from the same logits (layers.cu:1351-1460,
host_sampling.cc:114-146).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = torch.device(device)

    def __call__(self, logits: torch.Tensor, rows: Sequence) -> torch.Tensor:
        """``rows``: objects with temperature, top_p, top_k, min_p, seed, and optionally
        the penalties, ``history``, ``masked`` (one per logits row).  Returns int32 ids on
        the device; ``logits`` is changed where a row has penalties or masked tokens."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} logits rows for {len(rows)} sampling rows")
        self._penalise(logits, rows)
        if all(not (r.temperature > 0) for r in rows):
            return self.ops.sample(logits)
        dev = self.device
        temp = torch.tensor([float(r.temperature) for r in rows], dtype=torch.float32, device=dev)
        seeds = torch.tensor([_signed64(r.seed) for r in rows], dtype=torch.int64, device=dev)
        top_p = top_k = min_p = None
        if any(r.top_p < 1.0 for r in rows):
            top_p = torch.tensor([float(r.top_p) for r in rows], dtype=torch.float32, device=dev)
        if any(r.top_k > 0 for r in rows):
            top_k = torch.tensor([int(r.top_k) for r in rows], dtype=torch.int32, device=dev)
        if any(r.min_p > 0 for r in rows):
            min_p = torch.tensor([float(r.min_p) for r in rows], dtype=torch.float32, device=dev)
        return self.ops.sample(logits, temp, seeds, top_p=top_p, top_k=top_k, min_p=min_p)

    def _penalise(self, logits: torch.Tensor, rows: Sequence) -> None:
        hist = [getattr(r, "history", ()) for r in rows]
        masks = [getattr(r, "masked", ()) for r in rows]
        has_hist, has_mask = any(hist), any(masks)
        if not has_hist and not has_mask:
            return
        dev = self.device
        ids = counts = pen = mask = None
        if has_hist:
            cap = max(len(h) for h in hist)
            ids_h = torch.full((len(rows), cap), -1, dtype=torch.int32)
            counts_h = torch.zeros((len(rows), cap), dtype=torch.int32)
            pen_h = torch.zeros((len(rows), 3), dtype=torch.float32)
            for i, (r, h) in enumerate(zip(rows, hist)):
                pen_h[i, 2] = 1.0
                if h:
                    ids_h[i, :len(h)] = torch.tensor([t for t, _ in h], dtype=torch.int32)
                    counts_h[i, :len(h)] = torch.tensor([c for _, c in h], dtype=torch.int32)
                    pen_h[i] = torch.tensor([r.presence_penalty, r.frequency_penalty,
                                             r.repetition_penalty])
            ids, counts, pen = ids_h.to(dev), counts_h.to(dev), pen_h.to(dev)
        if has_mask:
            cap = max(len(m) for m in masks)
            mask_h = torch.full((len(rows), cap), -1, dtype=torch.int32)
            for i, m in enumerate(masks):
                if m:
                    mask_h[i, :len(m)] = torch.tensor(list(m), dtype=torch.int32)
            mask = mask_h.to(dev)
        self.ops.apply_penalties(logits, ids, counts, pen, mask)

    def logprobs(self, logits: torch.Tensor, ids: torch.Tensor, rows: Sequence):
        """For the rows that asked (``logprobs_k >= 0``): device tensors (chosen_lp [R],
        top_ids [R,K], top_lps [R,K]) and the per-row counts, or None when no row asked.
        ``logits`` are the ones the tokens were chosen from."""
        ks = [int(getattr(r, "logprobs_k", -1)) for r in rows]
        if all(k < 0 for k in ks):
            return None
        top = max(0, max(ks))
        want = torch.tensor(ks, dtype=torch.int32, device=self.device)
        chosen_lp, top_ids, top_lps = self.ops.token_logprobs(logits, ids, want, top)
        return chosen_lp, top_ids, top_lps, ks


def _signed64(u: int) -> int:
    u &= (1 << 64) - 1
    return u - (1 << 64) if u >= (1 << 63) else u
