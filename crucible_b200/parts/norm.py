"""RMSNorm: y_i = x_i * rsqrt(mean(x^2) + eps) * gain_i, scale first, then gain.

Formula and order: `model.py:113-118` (whole norm in fp32, gain multiplied in
fp32), `engine/kernels/kernels.cu:143-157`.  The input is the fp32 residual
stream; the statistics and both multiplications are 32-bit in either engine
dtype, and only the result is rounded to the engine dtype.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import small_batch
from ..config.model_config import NormSpec
from .base import NORMS, Norm, TensorDecl


class RMSNorm(Norm):
    def __init__(self, spec: NormSpec):
        self.spec = spec
        self.gain = None
        self.dtype = None

    def tensors(self):
        return [TensorDecl("gain", (self.spec.width,), role="vector")]

    def bind(self, tensors, dtype, device):
        self.gain = tensors["gain"]
        self.dtype = dtype

    supports_lazy = True
    supports_ahead = True      # the product that writes the rows last may leave this norm's input

    def forward(self, ctx, x: torch.Tensor, lazy: bool = False):
        """`lazy`: the consumer can fuse the normalisation into its first matrix
        product; for steps of a few rows it then gets the rows not yet normalised
        (`ops.small_batch.LazyNorm`) instead of a tensor."""
        def run():
            out = ctx.scratch("norm.out", (x.shape[0], self.spec.width), self.dtype)
            ops.rmsnorm(x, self.gain, self.spec.eps, out)
            return out
        take = getattr(ctx, "take_prenormed", None)
        pre = take(x, self) if take is not None else None
        if lazy and self.dtype == torch.bfloat16 and pre is not None:
            scaled, sumsq, parts = pre
            return small_batch.LazyNorm(x, self.gain, self.spec.eps, run, scaled, sumsq, parts)
        if lazy and self.dtype == torch.bfloat16 and x.shape[0] <= small_batch.MAX_LAZY_ROWS:
            return small_batch.LazyNorm(x, self.gain, self.spec.eps, run)
        return run()


NORMS.register("rmsnorm", RMSNorm)
