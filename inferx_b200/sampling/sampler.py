"""Turns a step's logits into token ids on the device.

One kernel launch per step for all rows: greedy rows (temperature <= 0) take the
argmax with ties to the lower index (src/backends/cuda/ops/layers.cu:413-452); the
others draw from softmax(logits / t) restricted by top-k, min-p and top-p with one
uniform keyed by the row's seed (layers.cu:1051-1303).  A batch that is all greedy
skips the parameter upload.
"""
from __future__ import annotations

from typing import Sequence

import torch


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = torch.device(device)

    def __call__(self, logits: torch.Tensor, rows: Sequence) -> torch.Tensor:
        """``rows``: objects with temperature, top_p, top_k, min_p, seed (one per logits
        row).  Returns int32 ids on the device."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} logits rows for {len(rows)} sampling rows")
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


def _signed64(u: int) -> int:
    u &= (1 << 64) - 1
    return u - (1 << 64) if u >= (1 << 63) else u
