"""The Python entry point: `LLM(model_dir).generate(prompts, params)`.

Token ids in, token ids out (the reference's tokenizer is outside this engine's
contract).  Option names and meanings follow the reference's command line where
it has them (`engine/src/main.rs:130-160`, `:476-497`): `max_batch`, `kv_pages`,
`prefill_chunk_tokens`, `prefill_token_budget`, `max_prefill_requests`, `graph`;
`profile=True` attributes device time to the model's parts (`engine/profile.py`).
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Union

from ..sampling.params import SamplingParams
from .engine import Engine, EngineOptions
from .scheduler import Completion, Request, Scheduler, SchedulerOptions


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_batch: int = 16, kv_pages: Optional[int] = None, page_tokens: int = 16,
                 prefill_token_budget: int = 1024, prefill_chunk_tokens: Optional[int] = None,
                 max_prefill_requests: Optional[int] = None, graph: bool = True,
                 profile: bool = False):
        self.engine = Engine(model, EngineOptions(dtype=dtype, page_tokens=page_tokens,
                                                  n_pages=kv_pages, max_requests=max_batch,
                                                  device=device, graph=graph, profile=profile))
        self.scheduler_options = SchedulerOptions(
            max_batch=max_batch, prefill_token_budget=prefill_token_budget,
            prefill_chunk_tokens=prefill_chunk_tokens, max_prefill_requests=max_prefill_requests)
        self.last_steps = []

    @property
    def config(self):
        return self.engine.config

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 ) -> List[List[int]]:
        """Generates for every prompt; returns the new token ids per prompt, in
        the order of `prompts`."""
        if params is None:
            params = SamplingParams()
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt is needed")
        sched = Scheduler(self.engine, self.scheduler_options)
        for i, (prompt, p) in enumerate(zip(prompts, params)):
            sched.submit(Request(i, list(prompt), p))
        self.last_steps = []
        done = {}
        try:
            while sched.has_work():
                t0 = time.perf_counter()
                info = sched.step()
                info.wall_s = time.perf_counter() - t0
                self.last_steps.append(info)
                if info.batch_tokens == 0 and info.admitted == 0 and info.finished == 0:
                    raise RuntimeError("generation made no progress")
                for c in sched.done:
                    done[c.id] = c
                sched.done = []
            sched.flush()
            for c in sched.done:
                done[c.id] = c
            # every id came to the host with the status word behind it (`PendingIds.get`);
            # this last look also covers steps that chose nothing
            from ..ops import tensor_core
            tensor_core.check_status(self.engine.device)
        except Exception:
            sched.abort()          # the engine keeps nothing of a run that failed
            raise
        return [done[i].tokens for i in range(len(prompts))]
