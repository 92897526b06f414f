"""What every part sees: the build context, the per-step context, cache needs.

Interfaces (duck-typed; a part defined outside this package works the same):

* every part: ``__init__(spec, ctx: BuildContext, prefix: str)``,
  ``tensors() -> [TensorDecl]`` (full checkpoint names), ``bind(weights: dict)``
  (receives exactly the declared tensors, on the device, already converted).
* norm: ``forward(resid, delta, rows=None) -> normed``; adds ``delta`` into the
  fp32 residual in place (unless ``rows`` picks rows to gather) and returns the
  normalised activations in the run's element type.
* position encoding: ``rotary_table() -> (inv_freq fp32 [rotary_dim/2] | None,
  rotary_dim)``; optionally ``apply(q, k, positions)`` for encodings that are not
  a rotation table (called on dense q and k before k enters the cache).
* mixer: ``cache_needs() -> [PagedKvNeed | StateNeed]``,
  ``forward(x, step: StepContext, cache: LayerCache) -> [T, hidden]``.
* feed-forward: ``forward(x, step) -> [T, hidden]``.
* block (the arrangement of the parts of one layer): ``__init__(spec, ctx, prefix)``,
  ``parts() -> [part]``, ``cache_needs()``, ``forward(resid, pending, step, cache) ->
  pending`` on the fp32 residual stream (``pending`` is a contribution the next norm
  still has to add).

A part may also define ``check_limits()``; it is called when the model is built and
raises if a size is beyond what the kernels take, so that a model that cannot run is
refused before any weight is read rather than at its first launch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch


@dataclass
class BuildContext:
    dtype: torch.dtype          # element type of activations and matrices
    device: torch.device
    ops: Any                    # the kernel module (inferx_b200.kernels.ops)


@dataclass(frozen=True)
class PagedKvNeed:
    """A record per token, kept in pages.  ``entries`` names the tensors of the record:
    keys and values by default, a single name for a mixer that keeps one vector per
    token (the reference parameterises ``KvLayout.entries_per_token`` for this,
    include/inferx/core/kv_cache.h:22-38).  Each entry is stored as ``[pages, kv_heads,
    page_size, head_dim]`` in ``dtype`` (None: the run's element type).  ``window`` = 0
    keeps every token; otherwise pages wholly behind the last ``window`` tokens may be
    given back.  Layers with the same window share page numbers and block tables
    whatever their records look like: a page is a span of tokens, and every layer has
    tensors of its own behind the page numbers."""
    kv_heads: int
    head_dim: int
    window: int = 0
    entries: Tuple[str, ...] = ("k", "v")
    dtype: Optional[torch.dtype] = None

    def bytes_per_token(self, run_dtype: torch.dtype) -> int:
        esize = torch.empty((), dtype=self.dtype or run_dtype).element_size()
        return len(self.entries) * self.kv_heads * self.head_dim * esize


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (not per token), zeroed when a request
    gets its slot: ``[slots, *shape]`` of ``dtype``."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class GroupView:
    """One cache group's view of the step: where each sequence's pages are and
    where this step's tokens go."""
    block_table: torch.Tensor   # [S, max_blocks] int32, -1 where no page is held
    slots: torch.Tensor         # [T] int32: page * page_size + offset
    page_size: int
    window: int
    # host mirror: per sequence, the index of the first page still held (pages before it
    # were given back as the window passed them); None in a step recorded for replay
    first_live: Optional[List[int]] = None


@dataclass
class StepContext:
    """One batch: tokens of several sequences, grouped by sequence in ascending
    sequence index with contiguous positions inside a sequence."""
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor     # [T] int32
    positions: torch.Tensor     # [T] int32
    seq_of_token: torch.Tensor  # [T] int32
    cu_q: torch.Tensor          # [S+1] int32: token range of each sequence
    q_pos0: torch.Tensor        # [S] int32: position of each sequence's first token here
    kv_len: torch.Tensor        # [S] int32: tokens each sequence holds after this step
    state_slot: torch.Tensor    # [S] int32
    groups: List[GroupView]
    max_q_len: int
    max_kv_len: int
    # Host mirrors, for parts that need loop bounds or launch shapes.  ``q_lens``,
    # ``num_decode_seqs`` and the width of each block table are the *shape* of a step:
    # they hold for every replay of a recorded step.  ``kv_lens``, ``state_slots`` and
    # each group's ``first_live`` are *values* of one step; when the step is recorded
    # into a CUDA graph (``captured``) they are None, and a part must index with the
    # device tensors (``kv_len``, ``state_slot``, ``block_table``) instead, which the
    # replay refreshes.  ``max_kv_len`` is then an upper bound for the shape.
    q_lens: List[int] = field(default_factory=list)
    kv_lens: Optional[List[int]] = None
    state_slots: Optional[List[int]] = None
    captured: bool = False
    all_decode: bool = False
    # Sequences that bring a single token come first in the batch: the first
    # ``num_decode_seqs`` sequences (and tokens).  ``cu_q_prompt`` is ``cu_q`` of the
    # remaining sequences counted from their own first token, so that a mixer can hand
    # the two parts of a mixed batch to different kernels without gathering.
    num_decode_seqs: int = 0
    cu_q_prompt: Optional[torch.Tensor] = None   # [S - num_decode_seqs + 1] int32


@dataclass
class LayerCache:
    """What one run of a layer gets from the cache: the paged tensors of the layer it
    reads (its own unless the schedule says otherwise) by entry name, the group whose
    block table addresses them, and per-request state tensors by name."""
    group: int = -1
    pages: Dict[str, torch.Tensor] = field(default_factory=dict)  # [pages, heads, page, dim]
    writes: bool = True
    state: Dict[str, torch.Tensor] = field(default_factory=dict)

    @property
    def k(self) -> Optional[torch.Tensor]:
        return self.pages.get("k")

    @property
    def v(self) -> Optional[torch.Tensor]:
        return self.pages.get("v")
