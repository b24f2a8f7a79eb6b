"""The hand-over between a product that writes the residual rows last and the norm that reads
them next (`StepContext.announce_norm`, `offer_prenormed`, `take_prenormed`): who may take
what, without a GPU."""
import torch

from crucible_b200.engine.context import StepContext
from crucible_b200.parts.block import PreNormBlock


def _ctx():
    return StepContext.__new__(StepContext)        # the hand-over needs nothing of a step's layout


def test_an_offer_is_taken_once_by_the_norm_it_was_made_for():
    ctx, rows, other = _ctx(), torch.zeros(5, 8), torch.zeros(5, 8)
    norm_a, norm_b = object(), object()
    assert ctx.norm_ahead(rows) is None and ctx.take_prenormed(rows, norm_a) is None
    ctx.announce_norm(norm_a, rows)
    assert ctx.norm_ahead(other) is None           # other rows
    assert ctx.norm_ahead(rows[:4]) is None        # the same memory, another shape
    assert ctx.norm_ahead(rows) is norm_a
    ctx.offer_prenormed(rows, norm_a, "scaled", "sumsq", 3)
    assert ctx.norm_ahead(rows) is None            # honoured: nobody else is asked
    assert ctx.take_prenormed(rows, norm_b) is None        # another norm gets nothing, and the offer is gone
    assert ctx.take_prenormed(rows, norm_a) is None
    ctx.announce_norm(norm_a, rows)
    ctx.offer_prenormed(rows, norm_a, "scaled", "sumsq", 3)
    assert ctx.take_prenormed(other, norm_a) is None
    ctx.announce_norm(norm_a, rows)
    ctx.offer_prenormed(rows, norm_a, "scaled", "sumsq", 3)
    assert ctx.take_prenormed(rows, norm_a) == ("scaled", "sumsq", 3)
    assert ctx.take_prenormed(rows, norm_a) is None        # once


def test_a_new_announcement_withdraws_an_offer_nobody_took():
    ctx, rows = _ctx(), torch.zeros(3, 4)
    norm = object()
    ctx.announce_norm(norm, rows)
    ctx.offer_prenormed(rows, norm, "scaled", "sumsq", 1)
    ctx.announce_norm(None, None)
    assert ctx.take_prenormed(rows, norm) is None


def test_the_block_announces_only_what_both_sides_can_do():
    class Norm:
        supports_ahead = True

    class PlainNorm:
        pass

    class Fusing:
        fuses_norm = True

    class Ctx:
        def __init__(self):
            self.calls = []

        def announce_norm(self, norm, rows):
            self.calls.append(norm)
    rows, norm = torch.zeros(2, 2), Norm()
    ctx = Ctx()
    PreNormBlock._announce(ctx, (norm, Fusing()), rows)
    PreNormBlock._announce(ctx, (norm, object()), rows)          # the consumer wants normalised rows
    PreNormBlock._announce(ctx, (PlainNorm(), Fusing()), rows)   # a norm that has no such form
    PreNormBlock._announce(ctx, None, rows)                      # nothing follows
    assert ctx.calls == [norm, None, None, None]
    PreNormBlock._announce(object(), (norm, Fusing()), rows)     # a context without the hand-over
