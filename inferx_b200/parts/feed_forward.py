"""Feed-forward parts: the dense SwiGLU and the routed mixture of experts.

Dense (src/model/qwen2.cc:1042-1048, 1413-1434): gate and up fused along the
output dimension, ``silu(gate) * up``, down projection, no biases.

Mixture of experts (src/model/moe_ffn.cc:158-367): router logits -> softmax over
all experts -> top-k (ties to the lower index) -> optional renormalisation ->
routed scale; stable dispatch by expert; per expert ``down(silu(gate(x)) *
up(x))``; combine in slot order with fp32 weights; a shared expert over every
token whose output is scaled by ``sigmoid(x . w_gate)`` when gated
(moe_ffn.cc:308-355).  Expert weights are stacked per layer as
``[E, 2I, H]`` (gate rows then up rows per expert) and ``[E, H, I]``
(src/model/deepseek_v2.cc:519-556).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .registry import build_part, register_part


class SwiGluFeedForward:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.gate_up_w = self.down_w = None

    def tensors(self):
        s, p = self.spec, self.prefix
        return [
            TensorDecl(f"{p}.gate_proj.weight", (s.intermediate, s.hidden)),
            TensorDecl(f"{p}.up_proj.weight", (s.intermediate, s.hidden)),
            TensorDecl(f"{p}.down_proj.weight", (s.hidden, s.intermediate)),
        ]

    def bind(self, w):
        p = self.prefix
        self.gate_up_w = torch.cat([w[f"{p}.gate_proj.weight"], w[f"{p}.up_proj.weight"]],
                                   dim=0).contiguous()
        self.down_w = w[f"{p}.down_proj.weight"]

    def forward(self, x, step=None):
        ops = self.ctx.ops
        return ops.linear(ops.gate_up_swiglu(x, self.gate_up_w), self.down_w)


_SIDE_STREAMS: dict = {}


class MoeFeedForward:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        if spec.top_k > spec.num_experts:
            raise ValueError("top_k exceeds the number of experts")
        self.router_w = self.expert_gate_up = self.expert_down = None
        self.shared = None
        self._shared_bytes = 0
        self.shared_gate_w = None
        self._side = None
        if spec.shared is not None:
            # any registered feed-forward may serve as the shared expert
            self.shared = build_part("feed_forward", spec.shared, ctx,
                                     f"{prefix}.{spec.shared_name}")

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_router_limits", None)
        if check is not None:
            check(self.spec.hidden, self.spec.num_experts, self.spec.top_k, self.prefix)
        if self.shared is not None and hasattr(self.shared, "check_limits"):
            self.shared.check_limits()

    def tensors(self):
        s, p = self.spec, self.prefix
        decls = [TensorDecl(f"{p}.gate.weight", (s.num_experts, s.hidden), keep="float32")]
        for e in range(s.num_experts):
            decls += [
                TensorDecl(f"{p}.experts.{e}.gate_proj.weight", (s.expert_intermediate, s.hidden)),
                TensorDecl(f"{p}.experts.{e}.up_proj.weight", (s.expert_intermediate, s.hidden)),
                TensorDecl(f"{p}.experts.{e}.down_proj.weight", (s.hidden, s.expert_intermediate)),
            ]
        if self.shared is not None:
            decls += self.shared.tensors()
            if s.shared_gated:
                decls.append(TensorDecl(f"{p}.{s.shared_gate_name}.weight", (1, s.hidden),
                                        keep="float32"))
        return decls

    def bind(self, w):
        s, p = self.spec, self.prefix
        self.router_w = w[f"{p}.gate.weight"]
        gu = torch.empty((s.num_experts, 2 * s.expert_intermediate, s.hidden),
                         dtype=self.ctx.dtype, device=self.ctx.device)
        dn = torch.empty((s.num_experts, s.hidden, s.expert_intermediate),
                         dtype=self.ctx.dtype, device=self.ctx.device)
        for e in range(s.num_experts):
            gu[e, :s.expert_intermediate] = w[f"{p}.experts.{e}.gate_proj.weight"]
            gu[e, s.expert_intermediate:] = w[f"{p}.experts.{e}.up_proj.weight"]
            dn[e] = w[f"{p}.experts.{e}.down_proj.weight"]
        self.expert_gate_up, self.expert_down = gu, dn
        if self.shared is not None:
            self.shared.bind({d.name: w[d.name] for d in self.shared.tensors()})
            self._shared_bytes = sum(w[d.name].numel() * w[d.name].element_size()
                                     for d in self.shared.tensors())
            if s.shared_gated:
                self.shared_gate_w = w[f"{p}.{s.shared_gate_name}.weight"].reshape(-1).contiguous()

    # In a step of few tokens the kernels leave the GPU partly idle; the shared
    # expert (which needs nothing from the router) then runs beside the routed experts,
    # on a stream of its own: its products cover the router's short kernels and the
    # boundaries between them (69 MB of shared weights a layer: a decode step of 3.94
    # against 4.27 ms at batch 8, 13.4 against 13.5 ms at batch 64).  One case is left
    # out: a large shared expert in a step of a few tokens, where its products and the
    # routed ones are the same kind of weight-streaming kernel, each able to keep the
    # memory busy alone, and beside each other they only take each other's places on the
    # multiprocessors (440 MB of shared weights a layer at batch 8: 19.3 ms beside, 16.1 ms
    # after; at batch 1, where the routed products are short, 6.1 beside against 6.6 ms,
    # and at batch 32, where the routed products are persistent tensor-core kernels, 24.7
    # against 25.4 ms).  Swapping the roles there - the shared expert on the main stream,
    # the router's short kernels and the dispatch beside it - measured worse still (20.1 ms).
    #
    # In larger steps the shared expert still runs on the stream of its own, but it
    # is handed over later, after the dispatch and just before the routed gate/up product:
    # at prompt sizes the routed products are bound by reading the experts' weights and
    # leave the tensor pipe idle, the shared expert's products are bound by the tensor
    # pipe, and the routed kernels, launched first, keep their places (a prompt portion of
    # 512 tokens 5.0 against 5.6 ms, 1,024 tokens 7.1 against 7.6 ms, 2,048 tokens 12.26
    # against 12.55 ms, 8,192 tokens 44.6 against 45.0 ms; handed over first, as below the
    # bound, 5.5 / 7.2 / 12.1 / 45.5 ms).  Not for a large shared expert: at the sizes that
    # have one (64 experts of 2560 x 3584, eight chosen) an expert sees 256 rows of a
    # 2,048-token portion and the routed products keep the tensor pipe busy themselves
    # (62.5 against 62.7 ms), while what the shared expert allocates on its own stream (a
    # gigabyte at 8,192 tokens and 20,480 columns) comes on top of what the main stream
    # holds, since the allocator keeps a pool per stream.
    # Between the two the later hand-over already pays (128 tokens 3.84 against 4.18 ms,
    # 256 tokens 4.19 against 4.55 ms; 32 tokens and decode steps of 32 and 64 sequences the
    # same either way), so the early one is kept for steps of at most 16 tokens, and, for a
    # large shared expert, which is never handed over late, up to 256.
    OVERLAP_MAX_TOKENS = 256
    EARLY_MAX_TOKENS = 16
    OVERLAP_LARGE_WEIGHT_BYTES = 160 << 20
    OVERLAP_LARGE_NOT_FOR_TOKENS = (3, 16)

    def _overlap_shared(self, tokens: int) -> bool:
        """Whether the shared expert is handed to its stream before the router."""
        large = self._shared_bytes > self.OVERLAP_LARGE_WEIGHT_BYTES
        if tokens > (self.OVERLAP_MAX_TOKENS if large else self.EARLY_MAX_TOKENS):
            return False
        lo, hi = self.OVERLAP_LARGE_NOT_FOR_TOKENS
        return not (large and lo <= tokens <= hi)

    def _side_stream(self):
        # One stream per device for all layers: the allocator keeps a pool of memory per
        # stream, and a stream per layer kept every layer's copy of the shared expert's
        # activations for itself (7 GB at 8,192 tokens and 24 layers); the layers run one
        # after the other anyway.
        if self._side is None:
            dev = torch.device(self.ctx.device)
            if dev not in _SIDE_STREAMS:
                _SIDE_STREAMS[dev] = torch.cuda.Stream(device=dev)
            self._side = _SIDE_STREAMS[dev]
        return self._side

    def forward(self, x, step=None):
        s, ops = self.spec, self.ctx.ops
        shared, side, ready = None, None, None
        beside = self.shared is not None and x.is_cuda
        if beside and self._overlap_shared(x.shape[0]):
            side = self._side_stream()
            main = torch.cuda.current_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared = self.shared.forward(x, step)
        elif (beside and x.shape[0] > self.EARLY_MAX_TOKENS
              and self._shared_bytes <= self.OVERLAP_LARGE_WEIGHT_BYTES):
            side = self._side_stream()
            main = torch.cuda.current_stream(x.device)
            ready = main.record_event()        # x is there; what follows is not waited for
        topk_w, topk_idx, shared_logit = ops.router_topk(
            x, self.router_w, s.top_k, s.renormalize, s.routed_scale, extra_w=self.shared_gate_w)
        offsets, rows, dest = ops.moe_dispatch(topk_idx, s.num_experts)
        if ready is not None:
            side.wait_event(ready)
            with torch.cuda.stream(side):
                shared = self.shared.forward(x, step)
        act = ops.grouped_gate_up_swiglu(x, rows, offsets, self.expert_gate_up)
        # `offsets` was written by the dispatch, two launches back: the down product may
        # start on its weights while the gate/up product drains
        y = ops.grouped_down(act, offsets, self.expert_down, offsets_settled=True)
        if side is not None:
            main.wait_stream(side)
        elif self.shared is not None:
            shared = self.shared.forward(x, step)
        combine = getattr(ops, "moe_combine_pending", ops.moe_combine)
        return combine(y, dest, topk_w, shared, shared_logit)


register_part("feed_forward", "swiglu", SwiGluFeedForward)
register_part("feed_forward", "moe", MoeFeedForward)
