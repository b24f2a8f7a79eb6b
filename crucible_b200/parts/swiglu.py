"""Dense SwiGLU feed-forward: x += (silu(n Wg^T) * (n Wu^T)) Wd^T.

`model.py:240-245`, `engine/src/model.rs:254-273`; SiLU on the gate,
g / (1 + exp(-g)), in fp32 (`engine/kernels/kernels.cu:1038-1047`).  Gate and
up matrices are stored separately in the checkpoint and concatenated at load
into one [2I, d] operand so one matrix product serves both; each output element
is still the same dot product, so numerics per element do not change.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.model_config import FeedForwardSpec
from .base import FEED_FORWARDS, FeedForward, TensorDecl


class SwiGLU(FeedForward):
    fuses_norm = True

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec
        self.gate_up = None
        self.down = None
        self.dtype = None

    def tensors(self):
        d, i = self.spec.width, self.spec.intermediate
        return [TensorDecl("gate", (i, d)), TensorDecl("up", (i, d)), TensorDecl("down", (d, i))]

    def bind(self, tensors, dtype, device):
        self.gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.down = tensors["down"]
        ops.declare_weights(self.gate_up, self.down)
        self.dtype = dtype

    def forward(self, ctx, h, residual):
        t, i = h.shape[0], self.spec.intermediate
        act = ctx.scratch("ffn.act", (t, i), self.dtype)
        ops.linear_swiglu(h, self.gate_up, act, ctx)
        ops.linear(act, self.down, residual, accumulate=True, closes=ctx)


FEED_FORWARDS.register("swiglu", SwiGLU)
