"""Block arrangements.  `pre_norm` is the only one the reference runs on the
GPU (`model.py:262-264`, `engine/src/gpu_model.rs:518-520`):
x = x + mixer(norm(x)); x = x + ffn(norm(x))."""
from __future__ import annotations

from .base import ARRANGEMENTS, Arrangement


class PreNormBlock(Arrangement):
    norm_names = ("mixer_norm", "feed_forward_norm")

    def forward(self, ctx, x, binding):
        h = self._norm(ctx, self.norms["mixer_norm"], self.mixer, x)
        self._announce(ctx, (self.norms["feed_forward_norm"], self.feed_forward), x)
        self.mixer.forward(ctx, h, x, binding)
        h = self._norm(ctx, self.norms["feed_forward_norm"], self.feed_forward, x)
        self._announce(ctx, getattr(ctx, "norm_after_layer", None), x)
        self.feed_forward.forward(ctx, h, x)

    def entry_norm(self):
        """(norm, its consumer): the first reader of the rows this layer is given."""
        return self.norms["mixer_norm"], self.mixer

    @staticmethod
    def _announce(ctx, ahead, x):
        # the part that runs now writes x last before `ahead`'s norm reads it: its last product
        # may leave that norm's input (StepContext.announce_norm)
        announce = getattr(ctx, "announce_norm", None)
        if announce is None:
            return
        norm, consumer = ahead if ahead is not None else (None, None)
        if (norm is not None and getattr(consumer, "fuses_norm", False)
                and getattr(norm, "supports_ahead", False)):
            announce(norm, x)
        else:
            announce(None, None)

    @staticmethod
    def _norm(ctx, norm, consumer, x):
        # a consumer that can fuse the norm into its first product (`fuses_norm`)
        # may be handed rows that are not yet normalised, if the norm offers that
        if getattr(consumer, "fuses_norm", False) and getattr(norm, "supports_lazy", False):
            return norm.forward(ctx, x, lazy=True)
        return norm.forward(ctx, x)


ARRANGEMENTS.register("pre_norm", PreNormBlock)
