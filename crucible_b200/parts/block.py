"""Block arrangements.  `pre_norm` is the only one the reference runs on the
GPU (`model.py:262-264`, `engine/src/gpu_model.rs:518-520`):
x = x + mixer(norm(x)); x = x + ffn(norm(x))."""
from __future__ import annotations

from .base import ARRANGEMENTS, Arrangement


class PreNormBlock(Arrangement):
    def forward(self, ctx, x, binding):
        h = self.mixer_norm.forward(ctx, x)
        self.mixer.forward(ctx, h, x, binding)
        h = self.feed_forward_norm.forward(ctx, x)
        self.feed_forward.forward(ctx, h, x)


ARRANGEMENTS.register("pre_norm", PreNormBlock)
