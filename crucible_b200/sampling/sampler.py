"""Token selection for the rows of a step, on the device.

All rows greedy: the argmax kernels.  Otherwise one kernel that handles greedy
and sampled rows side by side; the host draws one uniform number per sampled
row from that request's own generator and uploads it with the row's
temperature and top-k.  Only the chosen ids come back to the host, either at
once or, deferred, through a ring of pinned buffers while the next step already
runs (the ids then also stay on the device, per state slot, for that next step).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from .params import SamplingParams
from .rng import Xorshift64Star


class PendingIds:
    """Ids on their way to the host.  Behind them rides the status word of the
    tensor-core kernels as it stood when the ids were chosen: `get()` raises
    `KernelGaveUp` if a kernel of that step, or of one before it, ran out a bounded wait
    (its logits, and so these ids, are then not valid)."""

    def __init__(self, host: torch.Tensor, n: int, event: torch.cuda.Event, device=None):
        self._host, self._n, self._event, self._device = host, n, event, device
        self._ids: Optional[List[int]] = None

    def get(self) -> List[int]:
        if self._ids is None:
            self._event.synchronize()
            values = self._host[:self._n + 1].tolist()
            if self._device is not None and values[self._n]:
                from ..ops import tensor_core
                tensor_core.raise_if_gave_up(self._device, values[self._n])
            self._ids = values[:self._n]
        return self._ids


class Sampler:
    RING = 4

    def __init__(self, device, vocab: int):
        self.device = device
        self.vocab = vocab
        self._cap = 0
        self._at = 0
        self._copies = None          # the stream the ids travel to the host on

    def _buffers(self, n: int):
        if n > self._cap:
            cap = max(n, 64)
            torch.cuda.current_stream().synchronize()
            # per ring entry: pinned parameters [4, cap] (temperature, top-k bits, uniform,
            # slot bits), their device copy, device ids, pinned ids, and an event
            self._ring = [dict(host=torch.empty((4, cap), dtype=torch.float32, pin_memory=True),
                               dev=torch.empty((4, cap), dtype=torch.float32, device=self.device),
                               ids=torch.zeros(cap + 1, dtype=torch.int32, device=self.device),
                               ids_host=torch.zeros(cap + 1, dtype=torch.int32, pin_memory=True),
                               event=torch.cuda.Event(), chosen=torch.cuda.Event(), used=False)
                          for _ in range(self.RING)]
            self._cap = cap
        self._at = (self._at + 1) % self.RING
        slot = self._ring[self._at]
        if slot["used"]:
            slot["event"].synchronize()         # the copy that last read these buffers is done
        return slot

    def collect(self, ids: torch.Tensor, n: int, choice=None) -> PendingIds:
        """Ids that a step's own kernel has chosen (`ids`: n of them on the device, the status
        word behind them): sends them to the host on the copies' stream.  `choice`: whose
        buffers these are; it is told the event behind the copy, so that the step that writes
        them next can wait for it."""
        buf = self._buffers(n)
        if self._copies is None:
            self._copies = torch.cuda.Stream(device=self.device)
        buf["chosen"].record()
        self._copies.wait_event(buf["chosen"])
        ids.record_stream(self._copies)      # (an eager step's buffer may be freed before the copy runs)
        with torch.cuda.stream(self._copies):
            buf["ids_host"][:n + 1].copy_(ids[:n + 1], non_blocking=True)
            buf["event"].record(self._copies)
        buf["used"] = True
        if choice is not None:
            (choice.keeper or choice).copied = buf["event"]
        return PendingIds(buf["ids_host"], n, buf["event"], self.device)

    def sample(self, logits: torch.Tensor,
               rows: Sequence[Tuple[SamplingParams, Optional[Xorshift64Star]]],
               slots: Optional[Sequence[int]] = None,
               scatter_out: Optional[torch.Tensor] = None, defer: bool = False):
        """`logits`: fp32 [n, vocab] on the device; `rows[i]` = (params, generator).
        `slots`, `scatter_out`: also leave row i's id in scatter_out[slots[i]].
        Returns the ids, or with `defer` a `PendingIds`."""
        n = len(rows)
        if n == 0:
            return PendingIds(torch.zeros(1, dtype=torch.int32), 0, torch.cuda.Event()) if defer else []
        if logits.shape[0] != n:
            raise ValueError(f"{n} rows to sample but logits has {logits.shape[0]}")
        buf = self._buffers(n)
        ids = buf["ids"][:n]
        # the kernel that writes the ids also leaves the status word right behind them
        from ..ops import tensor_core
        status = (tensor_core.status_word(self.device), buf["ids"][n:n + 1])
        host = buf["host"].numpy()
        greedy = all(p.is_greedy for p, _ in rows)
        upload = not greedy or slots is not None
        scatter_index = None
        slots_fresh = False
        if slots is not None:
            # the slots of a running batch rarely change from step to step: each ring entry
            # remembers what its device copy holds and uploads the row only when it differs
            key = tuple(slots)
            slots_fresh = buf.get("slots") != key
            if slots_fresh:
                host[3, :n] = np.asarray(slots, dtype=np.int32).view(np.float32)
                buf["slots"] = key
            scatter_index = buf["dev"][3, :n].view(torch.int32)
        max_k = 1
        if not greedy:
            topk_bits = np.zeros(n, dtype=np.int32)
            for i, (p, rng) in enumerate(rows):
                if p.is_greedy:
                    host[0, i], topk_bits[i], host[2, i] = 0.0, 1, 0.0
                else:
                    k = p.effective_top_k(self.vocab)
                    max_k = max(max_k, k)
                    host[0, i], topk_bits[i], host[2, i] = p.temperature, k, rng.next_f32()
            host[1, :n] = topk_bits.view(np.float32)
        if upload:
            # one copy of whole rows of the parameter block (a slice [:, :n] is strided, and a
            # strided host-to-device copy goes through a staging buffer and a copy kernel)
            first, last = (3, 4) if greedy else (0, 4 if slots_fresh else 3)
            if not greedy or slots_fresh:
                buf["dev"][first:last].copy_(buf["host"][first:last], non_blocking=True)
        out = scatter_out if slots is not None else None
        if greedy:
            ops.argmax_rows(logits, ids, scatter_index, out, status=status)
        else:
            ops.sample_rows(logits, buf["dev"][0, :n], buf["dev"][1, :n].view(torch.int32),
                            buf["dev"][2, :n], max_k, ids, scatter_index, out, status=status)
        # the ids' way to the host runs on a stream of its own, so that the next step's launches
        # do not queue behind the copy
        if self._copies is None:
            self._copies = torch.cuda.Stream(device=self.device)
        buf["chosen"].record()
        self._copies.wait_event(buf["chosen"])
        with torch.cuda.stream(self._copies):
            buf["ids_host"][:n + 1].copy_(buf["ids"][:n + 1], non_blocking=True)
            buf["event"].record(self._copies)
        buf["used"] = True
        pending = PendingIds(buf["ids_host"], n, buf["event"], self.device)
        return pending if defer else pending.get()
