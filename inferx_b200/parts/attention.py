"""Grouped-query attention over the paged cache.

The reference's layer body (src/model/qwen2.cc:912-1030): one fused QKV
projection (weights concatenated in q, k, v order, qwen2.cc:1368-1403), biases on
Q, K and V only, rotation of Q and K after the bias, rotated keys written to the
cache before attention (qwen2.cc:928-931), scores scaled by a constant given in
the spec, causal by position with an optional window, and an output projection
without bias.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import PagedKvNeed
from .registry import build_part, register_part


class AttentionMixer:
    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        self.ctx = ctx
        self.prefix = prefix
        self.position = build_part("position", spec.position, ctx, prefix)
        self.qkv_w = self.qkv_b = self.o_w = None

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_attention_limits", None)
        if check is not None:
            s = self.spec
            check(s.heads, s.kv_heads, s.head_dim, self.ctx.dtype, self.prefix)

    # -- weights -----------------------------------------------------------
    def tensors(self):
        s, p = self.spec, self.prefix
        dq, dkv = s.heads * s.head_dim, s.kv_heads * s.head_dim
        decls = [
            TensorDecl(f"{p}.q_proj.weight", (dq, s.hidden)),
            TensorDecl(f"{p}.k_proj.weight", (dkv, s.hidden)),
            TensorDecl(f"{p}.v_proj.weight", (dkv, s.hidden)),
            TensorDecl(f"{p}.o_proj.weight", (s.hidden, dq)),
        ]
        if s.qkv_bias:
            decls += [
                TensorDecl(f"{p}.q_proj.bias", (dq,), keep="float32", init="bias"),
                TensorDecl(f"{p}.k_proj.bias", (dkv,), keep="float32", init="bias"),
                TensorDecl(f"{p}.v_proj.bias", (dkv,), keep="float32", init="bias"),
            ]
        if self.position is not None:
            decls += self.position.tensors()
        return decls

    def bind(self, w):
        p = self.prefix
        self.qkv_w = torch.cat([w[f"{p}.q_proj.weight"], w[f"{p}.k_proj.weight"],
                                w[f"{p}.v_proj.weight"]], dim=0).contiguous()
        self.o_w = w[f"{p}.o_proj.weight"]
        if self.spec.qkv_bias:
            self.qkv_b = torch.cat([w[f"{p}.q_proj.bias"], w[f"{p}.k_proj.bias"],
                                    w[f"{p}.v_proj.bias"]], dim=0).contiguous()
        if self.position is not None:
            self.position.bind(w)

    # -- cache -------------------------------------------------------------
    def cache_needs(self):
        return [PagedKvNeed(self.spec.kv_heads, self.spec.head_dim, self.spec.window)]

    # -- step --------------------------------------------------------------
    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        group = step.groups[cache.group]
        inv_freq, rot = (None, 0)
        if self.position is not None:
            inv_freq, rot = self.position.rotary_table()
        custom = getattr(self.position, "apply", None)
        fused = getattr(ops, "qkv_project_applies", None)
        if custom is None and cache.writes and fused is not None and fused(
                x, self.qkv_w, s.heads, s.kv_heads, s.head_dim, rot):
            # a few tokens: projection, bias, rotation and cache write in one kernel
            q = ops.qkv_project_rope_append(
                x, self.qkv_w, self.qkv_b, step.positions, inv_freq, rot, s.heads, s.kv_heads,
                s.head_dim, cache.k, cache.v, group.slots)
            attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window,
                                       s.scale)
            return ops.linear(attn.view(step.num_tokens, s.heads * s.head_dim), self.o_w)
        qkv = ops.linear(x, self.qkv_w)
        if custom is None:
            q = ops.qkv_rope_append(
                qkv, self.qkv_b, step.positions, inv_freq, rot, s.heads, s.kv_heads, s.head_dim,
                cache.k if cache.writes else None, cache.v if cache.writes else None,
                group.slots if cache.writes else None)
        else:
            # an encoding that is not a rotation table works on dense q and k first
            q, k, v = ops.qkv_rope_append(qkv, self.qkv_b, step.positions, None, 0, s.heads,
                                          s.kv_heads, s.head_dim, None, None, None,
                                          want_dense_kv=True)
            custom(q, k, step.positions)
            if cache.writes:
                ops.append_kv(k, v, cache.k, cache.v, group.slots)
        attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window, s.scale)
        return ops.linear(attn.view(step.num_tokens, s.heads * s.head_dim), self.o_w)


register_part("mixer", "attention", AttentionMixer)
