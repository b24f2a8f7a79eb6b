"""The continuous-batching scheduler above the step function.

States: pending -> prefilling -> active -> done (`engine/src/runtime.rs:96-125`,
`:177-198`).  One iteration: admit; build ONE mixed batch (every active
request's next token beside budgeted portions of prompts); run it; choose
tokens; retire.  The reference runs the decode call and the prefill plan as two
GPU calls per iteration (`runtime.rs:421-475`); here they are rows of one step.

Decisions, each from the reference:
 * admission is first come first served and stops at the first request that
   does not fit: no overtaking (`runtime.rs:490-535`); at most `max_batch`
   requests are resident (`:495`);
 * a request is admitted only if its whole lifetime, prompt + max_tokens - 1
   positions, can be reserved in every cache group (`prefill.rs:160-206`).
   So when pages run out the request WAITS in the queue (back-pressure,
   `runtime.rs:508-521`); a running request never meets an empty pool, nothing
   is preempted, swapped or recomputed.  A request that could never fit, or
   exceeds the context, is refused at submit (`prefill.rs:13-40`);
 * portions: each prefilling request is visited once per plan in queue order
   and gets min(remaining, chunk cap, budget left) tokens; unfinished ones go
   to the back of the queue (`prefill.rs:106-153`,
   `docs/packed-prefill-design.md:154-162`).  The budget is the step's token
   budget after the decoding rows have taken one token each;
 * the first token comes from the last prompt row's logits and the request's
   generator is created from its seed at that moment (`runtime.rs:722-744`);
 * a request finishes when it has max_tokens tokens (`runtime.rs:895`) or, an
   addition, when it produces its eos_token_id; its pages, reservation and
   state slot go back at once, between steps (`runtime.rs:896-898`);
 * cancel works in every state, between steps (`runtime.rs:923-960`).

The scheduler talks to an executor with five methods (`cache`, `add_request`,
`step`, `sample`, `finish`), so its decisions are tested on the CPU with a fake.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..sampling.params import SamplingParams
from ..sampling.rng import Xorshift64Star
from .engine import DEVICE_TOKEN, StepEntry

DEFAULT_PREFILL_TOKEN_BUDGET = 1024     # runtime.rs:208
DEFAULT_PREFILL_CHUNK = 128             # runtime.rs:205 (a cap; off unless asked for)


class SchedulerError(ValueError):
    pass


@dataclass
class SchedulerOptions:
    max_batch: int = 16
    prefill_token_budget: int = DEFAULT_PREFILL_TOKEN_BUDGET
    prefill_chunk_tokens: Optional[int] = None      # per-request cap on a portion
    max_prefill_requests: Optional[int] = None      # prompts sharing one step; default max_batch

    def validate(self) -> None:
        if self.max_batch <= 0:
            raise SchedulerError("max_batch must be positive")
        if self.prefill_token_budget <= 0:
            raise SchedulerError("prefill_token_budget must be positive")
        if self.prefill_chunk_tokens is not None and self.prefill_chunk_tokens <= 0:
            raise SchedulerError("prefill_chunk_tokens must be positive")
        if self.max_prefill_requests is not None and not (
                0 < self.max_prefill_requests <= self.max_batch):
            raise SchedulerError(f"max_prefill_requests must be in 1..={self.max_batch}")


@dataclass
class Request:
    id: Hashable
    prompt: Sequence[int]
    params: SamplingParams = field(default_factory=SamplingParams)


@dataclass
class Completion:
    id: Hashable
    prompt_len: int
    tokens: List[int]
    finish_reason: str            # "length", "eos" or "cancelled"


@dataclass
class _Live:
    request: Request
    done: int = 0                                  # prompt tokens already run
    generated: List[int] = field(default_factory=list)
    rng: Optional[Xorshift64Star] = None
    next_token: Optional[int] = None               # chosen, not yet run; None: still on the device
    n_chosen: int = 0                              # tokens chosen so far (known before their values)


@dataclass
class StepInfo:
    """What one iteration did (`runtime.rs:129-175`)."""
    step: int = 0
    admitted: int = 0
    decoded: int = 0
    prefill_tokens: int = 0
    prefill_requests: int = 0
    first_tokens: int = 0
    finished: int = 0
    batch_tokens: int = 0
    free_pages: List[int] = field(default_factory=list)
    pending: int = 0
    wall_s: float = 0.0           # host time of the iteration, filled in by the caller


class Scheduler:
    def __init__(self, executor, options: Optional[SchedulerOptions] = None):
        self.executor = executor
        self.options = options or SchedulerOptions()
        self.options.validate()
        self.pending: Deque[Request] = deque()
        self.prefilling: Deque[_Live] = deque()
        self.active: List[_Live] = []
        self.done: List[Completion] = []
        self.step_no = 0
        # Tokens chosen by the last step whose values have not reached the host yet:
        # (ids on their way, [(live, is_first_token), ...]).  With an executor that can
        # keep a request's latest token on the device (`sample_deferred`), a step is
        # queued before the previous step's ids are read, so the device never waits for
        # the host between steps; values are needed earlier only for eos_token_id.
        self._in_flight = None
        self._finishing: List[tuple] = []          # (live, reason) waiting for their last values

    # -- submission ---------------------------------------------------------------

    def _lifetime(self, request: Request) -> int:
        return len(request.prompt) + request.params.max_tokens - 1     # prefill.rs:160-171

    def _max_step_tokens(self) -> int:
        return self.options.prefill_token_budget

    def submit(self, request: Request) -> None:
        """Refuses malformed work before it can own pages (`runtime.rs:345-363`)."""
        ex = self.executor
        if len(request.prompt) == 0:
            raise SchedulerError("prompt length and output token budget must be positive")
        request.params.validate(ex.vocab_size, getattr(ex, "max_device_top_k", None))
        life = self._lifetime(request)
        if life > ex.max_context:
            raise SchedulerError(f"request needs {life} cache positions, capacity is "
                                 f"{ex.max_context}")
        if not ex.cache.fits_at_all(life, self._max_step_tokens()):
            raise SchedulerError(f"request needs more KV pages than the pool holds "
                                 f"({life} positions)")
        for tok in request.prompt:
            if not 0 <= int(tok) < ex.vocab_size:
                raise SchedulerError(f"request token {tok} outside vocabulary {ex.vocab_size}")
        live_ids = ([r.id for r in self.pending] + [l.request.id for l in self.prefilling]
                    + [l.request.id for l in self.active])
        if request.id in live_ids:
            raise SchedulerError(f"request id {request.id!r} is already queued or resident")
        self.pending.append(request)

    # -- one iteration ------------------------------------------------------------

    def has_work(self) -> bool:
        """Requests still to be run.  When this turns false, `flush()` brings in the
        last token values."""
        return bool(self.pending or self.prefilling or self.active)

    def step(self) -> StepInfo:
        info = StepInfo(step=self.step_no)
        self.step_no += 1
        info.admitted = self._admit()
        entries: List[StepEntry] = []
        sample_rows = []                     # (live, is_first_token)
        for live in self.active:
            token = live.next_token if live.next_token is not None else DEVICE_TOKEN
            entries.append(StepEntry(live.request.id, [token], [0]))
            sample_rows.append((live, False))
        info.decoded = len(self.active)
        plan = self._plan_prefill(budget=self.options.prefill_token_budget - len(self.active))
        for live, n in plan:
            tokens = live.request.prompt[live.done:live.done + n]
            final = live.done + n == len(live.request.prompt)
            entries.append(StepEntry(live.request.id, list(tokens), [n - 1] if final else []))
            if final:
                sample_rows.append((live, True))
            info.prefill_tokens += n
        info.prefill_requests = len(plan)
        info.batch_tokens = info.decoded + info.prefill_tokens
        if entries:
            # every entry chooses a token, greedily, and none can end on it: the choice is part
            # of the step (an executor that has `step_choosing` captures it with the step)
            choosing = (len(sample_rows) == len(entries) and hasattr(self.executor, "step_choosing")
                        and all(live.request.params.is_greedy and live.request.params.eos_token_id is None
                                for live, _ in sample_rows))
            if choosing:
                logits, chosen_ids = self.executor.step_choosing(entries)
            else:
                logits = self.executor.step(entries)
            rows = []
            for live, first in sample_rows:
                if first and not live.request.params.is_greedy:
                    live.rng = Xorshift64Star(live.request.params.seed)
                rows.append((live.request.params, live.rng))
            defer = (rows and hasattr(self.executor, "sample_deferred")
                     and all(p.eos_token_id is None for p, _ in rows))
            previous, self._in_flight = self._in_flight, None
            if defer:
                ids = chosen_ids if choosing else self.executor.sample_deferred(
                    logits, rows, [live.request.id for live, _ in sample_rows])
                for live, first in sample_rows:
                    live.n_chosen += 1
                    live.next_token = None
                    info.first_tokens += int(first)
                self._in_flight = (ids, list(sample_rows))
                self._resolve(previous)            # the step before: its ids have long arrived
            else:
                self._resolve(previous)
                chosen = self.executor.sample(logits, rows)
                for (live, first), tok in zip(sample_rows, chosen):
                    live.generated.append(int(tok))
                    live.next_token = int(tok)
                    live.n_chosen += 1
                    info.first_tokens += int(first)
        # bookkeeping of the prefill queue: finished prompts start decoding,
        # unfinished ones go to the back
        for live, n in plan:
            live.done += n
            self.prefilling.remove(live)
            if live.done == len(live.request.prompt):
                self.active.append(live)
            else:
                self.prefilling.append(live)
        info.finished = self._retire()
        info.free_pages = [self.executor.cache.free_pages(g)
                           for g in range(len(self.executor.cache.pools))]
        info.pending = len(self.pending)
        return info

    def _admit(self) -> int:
        n = 0
        while self.pending:
            if len(self.active) + len(self.prefilling) >= self.options.max_batch:
                break
            request = self.pending[0]
            life = self._lifetime(request)
            if not self.executor.cache.can_reserve(life, self._max_step_tokens()):
                break                                # waits; nobody overtakes it
            self.executor.add_request(request.id, life, self._max_step_tokens())
            self.pending.popleft()
            self.prefilling.append(_Live(request))
            n += 1
        return n

    def _plan_prefill(self, budget: int):
        limit = self.options.max_prefill_requests or self.options.max_batch
        cap = self.options.prefill_chunk_tokens
        plan, used = [], 0
        for live in self.prefilling:
            if len(plan) == limit or used >= budget:
                break
            remaining = len(live.request.prompt) - live.done
            n = min(remaining, budget - used)
            if cap is not None:
                n = min(n, cap)
            if n <= 0:
                break
            plan.append((live, n))
            used += n
        return plan

    def _resolve(self, in_flight) -> None:
        """Reads the values of tokens chosen earlier and files them."""
        if in_flight is None:
            return
        ids, rows = in_flight
        for (live, _), tok in zip(rows, ids.get()):
            live.generated.append(int(tok))
            if len(live.generated) == live.n_chosen:
                live.next_token = int(tok)
        still = []
        for live, reason in self._finishing:
            if len(live.generated) == live.n_chosen:
                self.done.append(Completion(live.request.id, len(live.request.prompt),
                                            live.generated, reason))
            else:
                still.append((live, reason))
        self._finishing = still

    def flush(self) -> None:
        """Waits for every token value still on its way."""
        previous, self._in_flight = self._in_flight, None
        self._resolve(previous)

    def _retire(self) -> int:
        n = 0
        i = 0
        while i < len(self.active):
            live = self.active[i]
            p = live.request.params
            reason = None
            if live.n_chosen >= p.max_tokens:
                reason = "length"
            elif (p.eos_token_id is not None and live.generated
                  and live.generated[-1] == p.eos_token_id):
                reason = "eos"
            if reason is None:
                i += 1
                continue
            # swap-remove: slot order changes on purpose; nothing is keyed on it
            self.active[i] = self.active[-1]
            self.active.pop()
            self.executor.finish(live.request.id)
            if len(live.generated) == live.n_chosen:
                self.done.append(Completion(live.request.id, len(live.request.prompt),
                                            live.generated, reason))
            else:
                self._finishing.append((live, reason))     # its last value is still on its way
            n += 1
        return n

    def cancel(self, request_id) -> bool:
        """Removes a request in any state; its pages and reservation go back."""
        for i, r in enumerate(self.pending):
            if r.id == request_id:
                del self.pending[i]
                self.done.append(Completion(request_id, len(r.prompt), [], "cancelled"))
                return True
        self.flush()
        for queue in (self.prefilling, self.active):
            for live in list(queue):
                if live.request.id == request_id:
                    queue.remove(live)
                    self.executor.finish(request_id)
                    self.done.append(Completion(request_id, len(live.request.prompt),
                                                live.generated, "cancelled"))
                    return True
        return False

    def abort(self) -> List[Hashable]:
        """After the executor failed in the middle of a run (`engine/src/server.rs:1187-1227`
        injects such a failure): every resident request gives back its pages, its
        reservation and its state slot, queued requests are dropped, and token values
        still on their way are forgotten.  Returns the ids of the requests it ended; the
        executor is then as empty as before the run."""
        ended = [r.id for r in self.pending]
        self.pending.clear()
        self._in_flight = None
        self._finishing = []
        for queue in (self.prefilling, self.active):
            for live in list(queue):
                ended.append(live.request.id)
                if self.executor.cache.has(live.request.id):
                    self.executor.finish(live.request.id)
            queue.clear()
        return ended

    def run_to_completion(self, max_steps: Optional[int] = None) -> List[Completion]:
        steps = 0
        try:
            while self.has_work():
                info = self.step()
                steps += 1
                if info.batch_tokens == 0 and info.admitted == 0 and info.finished == 0:
                    raise SchedulerError("the scheduler made no progress: a pending request "
                                         "cannot be admitted and nothing is running")
                if max_steps is not None and steps >= max_steps:
                    break
            self.flush()
        except Exception:
            self.abort()
            raise
        out, self.done = self.done, []
        return out
