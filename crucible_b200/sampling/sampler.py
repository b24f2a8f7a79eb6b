"""Token selection for the rows of a step, on the device.

All rows greedy: one argmax kernel.  Otherwise one kernel that handles greedy
and sampled rows side by side; the host draws one uniform number per sampled
row from that request's own generator and uploads it with the row's
temperature and top-k.  Only the chosen ids come back to the host.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from .params import SamplingParams
from .rng import Xorshift64Star


class Sampler:
    def __init__(self, device, vocab: int):
        self.device = device
        self.vocab = vocab
        self._cap = 0
        self._host = None
        self._dev = None
        self._ids = None
        self._ids_host = None

    def _buffers(self, n: int):
        if n > self._cap:
            cap = max(n, 64)
            self._host = torch.empty((3, cap), dtype=torch.float32, pin_memory=True)
            self._dev = torch.empty((3, cap), dtype=torch.float32, device=self.device)
            self._ids = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._ids_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._cap = cap

    def sample(self, logits: torch.Tensor,
               rows: Sequence[Tuple[SamplingParams, Optional[Xorshift64Star]]]) -> List[int]:
        """`logits`: fp32 [n, vocab] on the device; `rows[i]` = (params, generator)."""
        n = len(rows)
        if n == 0:
            return []
        if logits.shape[0] != n:
            raise ValueError(f"{n} rows to sample but logits has {logits.shape[0]}")
        self._buffers(n)
        ids = self._ids[:n]
        if all(p.is_greedy for p, _ in rows):
            ops.argmax_rows(logits, ids)
        else:
            host = self._host.numpy()
            max_k = 1
            topk_bits = np.zeros(n, dtype=np.int32)
            for i, (p, rng) in enumerate(rows):
                if p.is_greedy:
                    host[0, i], topk_bits[i], host[2, i] = 0.0, 1, 0.0
                else:
                    k = p.effective_top_k(self.vocab)
                    max_k = max(max_k, k)
                    host[0, i], topk_bits[i], host[2, i] = p.temperature, k, rng.next_f32()
            host[1, :n] = topk_bits.view(np.float32)
            self._dev[:, :n].copy_(self._host[:, :n], non_blocking=True)
            ops.sample_rows(logits, self._dev[0, :n], self._dev[1, :n].view(torch.int32),
                            self._dev[2, :n], max_k, ids)
        self._ids_host[:n].copy_(ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._ids_host[:n].tolist()
