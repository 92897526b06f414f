"""Rotary position encoding as a table of inverse frequencies.

Half-split (NeoX) pairing: for j < rotary_dim/2, ``inv_freq[j] = theta^(-2j /
rotary_dim)`` and the pair (x[j], x[j + rotary_dim/2]) is rotated by
``pos * inv_freq[j]`` (src/backends/cuda/ops/layers.cu:80-115).  The table is
computed once in float64 and rounded to fp32; the kernel forms the angle and its
sine and cosine in fp32.  Anything that can be written as such a table (scaled
frequencies, a partial rotary dimension, no rotation at all) reuses the fused
kernel by returning a different ``rotary_table()``.
"""
from __future__ import annotations

import torch

from .registry import register_part


class RotaryEncoding:
    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim < 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim "
                             f"{spec.head_dim}")
        half = spec.rotary_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64),
                        -2.0 * j / float(spec.rotary_dim))
        self.inv_freq = inv.to(torch.float32).to(ctx.device)

    def tensors(self):
        return []

    def bind(self, weights):
        pass

    def rotary_table(self):
        return (self.inv_freq if self.spec.rotary_dim else None), self.spec.rotary_dim


register_part("position", "rope", RotaryEncoding)
