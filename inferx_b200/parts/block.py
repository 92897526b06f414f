"""The decoder: blocks built from specs, run in the order a schedule gives.

A block is the pre-norm residual arrangement of the reference's layer body
(src/model/qwen2.cc:908-1051): ``x += mixer(norm(x)); x += ffn(norm(x))``.  The
residual stream ``x`` is fp32; each sub-part returns its contribution in the
run's element type and the following norm adds it in (one pass over the row
instead of the reference's copy + add + norm).  The decoder embeds, runs the
schedule's entries in order (a layer may appear twice, or read another layer's
cache), gathers the rows whose logits are wanted *before* the final norm, and
multiplies those rows by the head (the reference multiplies all rows,
src/model/qwen2.cc:1066).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..weights import loader as wl
from ..weights.loader import TensorDecl
from .base import BuildContext, LayerCache, StepContext
from .registry import build_part, register_part


class PreNormBlock:
    """``x += mixer(norm(x)); x += ffn(norm(x))`` on the fp32 residual stream."""

    def __init__(self, spec, ctx: BuildContext, prefix: str):
        p = prefix
        self.spec = spec
        self.input_norm = build_part("norm", spec.input_norm, ctx, f"{p}.{spec.input_norm_name}")
        self.mixer = build_part("mixer", spec.mixer, ctx, f"{p}.{spec.mixer_name}")
        self.post_norm = build_part("norm", spec.post_norm, ctx, f"{p}.{spec.post_norm_name}")
        self.ffn = build_part("feed_forward", spec.ffn, ctx, f"{p}.{spec.ffn_name}")

    def parts(self):
        return [self.input_norm, self.mixer, self.post_norm, self.ffn]

    def cache_needs(self):
        return list(self.mixer.cache_needs())

    def forward(self, resid, pending, step: StepContext, cache: LayerCache):
        """``pending`` is the previous block's contribution not yet added to
        ``resid``; returns this block's own pending contribution."""
        if hasattr(pending, "materialize") and not getattr(self.input_norm, "accepts_pending",
                                                            False):
            pending = pending.materialize()
        n = self.input_norm.forward(resid, pending)
        a = self.mixer.forward(n, step, cache)
        n = self.post_norm.forward(resid, a)
        return self.ffn.forward(n, step)


class DecoderModel:
    """Embedding, scheduled blocks, final norm and head, from a ``ModelSpec``."""

    def __init__(self, spec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        self.blocks = [build_part("block", ls, ctx, ls.prefix) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, ctx, spec.final_norm_name)
        self.embed = None
        self.head = None
        for e in spec.schedule:
            if not (0 <= e.layer < len(self.blocks)) or not (0 <= e.cache_layer < len(self.blocks)):
                raise ValueError(f"schedule entry {e} names a layer that does not exist")
        if ctx.ops is not None:
            # sizes beyond what the kernels take are refused now, not at the first launch
            for b in self.blocks:
                for part in b.parts():
                    if hasattr(part, "check_limits"):
                        part.check_limits()

    # -- weights -----------------------------------------------------------
    def _own_tensors(self) -> List[TensorDecl]:
        s = self.spec
        decls = [TensorDecl(s.embed_name, (s.vocab_size, s.hidden))]
        if not s.tied_head:
            decls.append(TensorDecl(s.head_name, (s.vocab_size, s.hidden)))
        return decls

    def tensors(self) -> List[TensorDecl]:
        decls = self._own_tensors()
        for b in self.blocks:
            for part in b.parts():
                decls += part.tensors()
        decls += self.final_norm.tensors()
        return decls

    def load(self, source: wl.WeightSource, where: str = "weights") -> None:
        """Check every declared tensor against the source, then bind part by part."""
        wl.check(self.tensors(), source, where)
        dt, dev = self.ctx.dtype, self.ctx.device

        def fetch(decls):
            return {d.name: wl.materialize(d, source, dt, dev) for d in decls}

        own = fetch(self._own_tensors())
        self.embed = own[self.spec.embed_name]
        self.head = self.embed if self.spec.tied_head else own[self.spec.head_name]
        for b in self.blocks:
            for part in b.parts():
                part.bind(fetch(part.tensors()))
        self.final_norm.bind(fetch(self.final_norm.tensors()))

    # -- cache needs -------------------------------------------------------
    def cache_needs(self) -> List[list]:
        """Per layer, what its mixer wants kept between steps."""
        return [list(b.cache_needs()) for b in self.blocks]

    # -- step --------------------------------------------------------------
    def forward(self, step: StepContext, caches: List[LayerCache],
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs the batch; returns fp32 logits [R, vocab] for ``logit_rows`` (token
        indices into the batch), or None when no logits are wanted."""
        ops = self.ctx.ops
        if hasattr(ops, "set_dependent_launch"):
            ops.set_dependent_launch(step.num_tokens <= ops.DEPENDENT_LAUNCH_MAX_TOKENS)
        resid = ops.embed(self.embed, step.token_ids)
        pending = None
        for entry, cache in zip(self.spec.schedule, caches):
            pending = self.blocks[entry.layer].forward(resid, pending, step, cache)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        if hasattr(pending, "materialize") and not getattr(self.final_norm, "accepts_pending",
                                                            False):
            pending = pending.materialize()
        n = self.final_norm.forward(resid, pending, rows=logit_rows)
        return ops.linear(n, self.head, out_dtype=torch.float32)


Block = PreNormBlock
register_part("block", "pre_norm", PreNormBlock)
