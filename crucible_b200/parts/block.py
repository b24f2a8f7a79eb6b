"""Block arrangements.  `pre_norm` is the only one the reference runs on the
GPU (`model.py:262-264`, `engine/src/gpu_model.rs:518-520`):
x = x + mixer(norm(x)); x = x + ffn(norm(x))."""
from __future__ import annotations

from .base import ARRANGEMENTS, Arrangement


class PreNormBlock(Arrangement):
    norm_names = ("mixer_norm", "feed_forward_norm")

    def forward(self, ctx, x, binding):
        h = self._norm(ctx, self.norms["mixer_norm"], self.mixer, x)
        self.mixer.forward(ctx, h, x, binding)
        h = self._norm(ctx, self.norms["feed_forward_norm"], self.feed_forward, x)
        self.feed_forward.forward(ctx, h, x)

    @staticmethod
    def _norm(ctx, norm, consumer, x):
        # a consumer that can fuse the norm into its first product (`fuses_norm`)
        # may be handed rows that are not yet normalised, if the norm offers that
        if getattr(consumer, "fuses_norm", False) and getattr(norm, "supports_lazy", False):
            return norm.forward(ctx, x, lazy=True)
        return norm.forward(ctx, x)


ARRANGEMENTS.register("pre_norm", PreNormBlock)
