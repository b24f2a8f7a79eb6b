"""Opt-in attribution of a step's device time to the model's parts.

With `EngineOptions(profile=True)` every part of the model (embedding, each
layer's norms, mixer and feed-forward, the final norm, the head) has its
`forward` bracketed by a pair of CUDA events on the launching stream; steps
then run eagerly (a captured step has no events to read).  `StageProfiler.table()`
waits for the device and returns, per stage, the number of calls, the total
milliseconds and the share of the whole.  When the option is off nothing is
wrapped and a step costs what it cost before.

A norm whose consumer fuses it (`ops.small_batch.LazyNorm`) runs inside the
consumer's first kernel, so its own row then shows next to nothing and the
consumer's row carries it.

The reference attributes stages the same way behind a compile-time switch
(`engine/src/gpu_model.rs:30-121`: a `const PROFILE` generic whose off form
compiles to nothing; `:2976-3041`: events around each stage of a prefill).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


class StageProfiler:
    def __init__(self):
        self._open: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self._totals: Dict[str, List[float]] = {}       # stage -> [calls, ms]
        self.steps = 0

    def wrap(self, part, stage: str) -> None:
        """Brackets `part.forward` with events filed under `stage`."""
        inner = part.forward

        def timed(*args, **kwargs):
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record()
            out = inner(*args, **kwargs)
            end.record()
            self._open.append((stage, start, end))
            return out
        part.forward = timed

    def _collect(self) -> None:
        if not self._open:
            return
        torch.cuda.synchronize()
        for stage, start, end in self._open:
            slot = self._totals.setdefault(stage, [0, 0.0])
            slot[0] += 1
            slot[1] += start.elapsed_time(end)
        self._open = []

    def reset(self) -> None:
        self._collect()
        self._totals = {}
        self.steps = 0

    def table(self) -> List[dict]:
        """[{stage, calls, ms, share}], largest first.  Synchronises."""
        self._collect()
        whole = sum(ms for _, ms in self._totals.values()) or 1.0
        rows = [{"stage": stage, "calls": calls, "ms": round(ms, 4), "share": round(ms / whole, 4)}
                for stage, (calls, ms) in self._totals.items()]
        rows.sort(key=lambda r: -r["ms"])
        return rows

    def text(self) -> str:
        rows = self.table()
        lines = [f"{'stage':28s} {'calls':>7s} {'ms':>10s} {'share':>7s}"]
        for r in rows:
            lines.append(f"{r['stage']:28s} {r['calls']:7d} {r['ms']:10.3f} {100 * r['share']:6.1f}%")
        lines.append(f"{'(steps)':28s} {self.steps:7d}")
        return "\n".join(lines)


def attach(model, profiler: StageProfiler) -> None:
    """Wraps every part of `model` (a `DecoderModel`): layers' parts are filed by their
    role in the layer and their kind, all layers together."""
    profiler.wrap(model.embedding, "embedding")
    profiler.wrap(model.final_norm, "final_norm")
    profiler.wrap(model.head, "head")
    for layer, spec in zip(model.layers, model.config.layers):
        for name, norm in layer.norms.items():
            profiler.wrap(norm, f"layer.{name}")
        profiler.wrap(layer.mixer, f"layer.mixer[{spec.mixer.kind}]")
        profiler.wrap(layer.feed_forward, f"layer.feed_forward[{spec.feed_forward.kind}]")
