"""RMSNorm with the residual add folded in.

``out = x * (1 / sqrt(mean(x^2) + eps)) * gain`` with the sum in fp32, no mean
subtraction, no bias, the gain used as stored (not 1 + gain): the reference's
RmsNormKernel (src/backends/cuda/ops/layers.cu:50-76).  The residual add that the
reference does in a kernel of its own (layers.cu:542-548) happens in the same
pass, on an fp32 residual stream.
"""
from __future__ import annotations

from ..weights.loader import TensorDecl
from .registry import register_part


class RmsNorm:
    # the contribution to add may arrive unwritten (``ops.CombinePending``); the kernel
    # behind ``add_rmsnorm`` folds it in
    accepts_pending = True

    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        self.ctx = ctx
        self.name = f"{prefix}.weight"
        self.gain = None

    def tensors(self):
        return [TensorDecl(self.name, (self.spec.size,), keep="float32", init="gain")]

    def bind(self, weights):
        self.gain = weights[self.name]

    def forward(self, resid, delta, rows=None):
        return self.ctx.ops.add_rmsnorm(resid, delta, self.gain, self.spec.eps, self.ctx.dtype,
                                        rows=rows)


register_part("norm", "rmsnorm", RmsNorm)
