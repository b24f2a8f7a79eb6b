"""The scheduler's decisions, on the CPU with a fake executor."""
from typing import List

import pytest

from crucible_b200.cache import CacheManager, GroupPolicy
from crucible_b200.engine.scheduler import (Request, Scheduler, SchedulerError, SchedulerOptions)
from crucible_b200.sampling import SamplingParams


class FakeExecutor:
    """Keeps a real cache manager; 'logits' are the list of (request, position)
    of the wanted rows; the chosen token is a function of those."""
    vocab_size = 1000
    max_context = 512

    def __init__(self, n_pages=16, page_tokens=16, max_requests=4):
        self.cache = CacheManager([GroupPolicy(page_tokens)], [n_pages], max_requests)
        self.steps: List[list] = []

    def add_request(self, request, lifetime_tokens=None, max_step_tokens=None):
        self.cache.add_request(request, lifetime_tokens, max_step_tokens)

    def step(self, entries):
        rows = []
        self.steps.append([(e.request, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            self.cache.extend(e.request, len(e.tokens))
            start = self.cache.length(e.request) - len(e.tokens)
            rows += [(e.request, start + w, e.tokens[w]) for w in e.want]
        self.cache.check_invariants()
        return rows

    def sample(self, logits, rows):
        assert len(logits) == len(rows)
        return [(pos * 7 + tok) % self.vocab_size for (_, pos, tok) in logits]

    def finish(self, request):
        self.cache.remove_request(request)


def greedy(n):
    return SamplingParams(max_tokens=n)


def test_prompts_are_cut_under_the_budget_and_decodes_ride_along():
    ex = FakeExecutor(n_pages=64)
    s = Scheduler(ex, SchedulerOptions(max_batch=4, prefill_token_budget=32))
    s.submit(Request("a", list(range(50)), greedy(3)))
    s.submit(Request("b", list(range(20)), greedy(2)))
    i0 = s.step()
    assert i0.admitted == 2 and ex.steps[0] == [("a", 32, [])]          # budget spent on a
    s.step()
    # a went to the back: b gets its 20 tokens first, then a gets the 12 left of the budget
    assert ex.steps[1] == [("b", 20, [19]), ("a", 12, [])]
    s.step()
    # b decodes (1 token) beside a's last portion; the budget left is 31
    assert ex.steps[2] == [("b", 1, [0]), ("a", 6, [5])]
    done = s.run_to_completion()
    by_id = {c.id: c for c in done}
    assert len(by_id["a"].tokens) == 3 and len(by_id["b"].tokens) == 2
    assert by_id["a"].finish_reason == "length"
    assert ex.cache.free_pages(0) == 64 and ex.cache.slots.free_slots == 4
    # positions used: prompt + max_tokens - 1
    assert sum(n for step in ex.steps for (r, n, _) in step if r == "a") == 50 + 3 - 1


def test_chunk_cap_and_request_limit():
    ex = FakeExecutor(n_pages=64)
    s = Scheduler(ex, SchedulerOptions(max_batch=4, prefill_token_budget=64,
                                       prefill_chunk_tokens=10, max_prefill_requests=2))
    for name in "abc":
        s.submit(Request(name, list(range(25)), greedy(1)))
    s.step()
    assert ex.steps[0] == [("a", 10, []), ("b", 10, [])]               # two prompts per step
    s.step()
    assert ex.steps[1] == [("c", 10, []), ("a", 10, [])]               # round robin
    s.run_to_completion()
    assert ex.cache.free_pages(0) == 64


def test_when_pages_run_out_the_request_waits_and_nobody_overtakes():
    ex = FakeExecutor(n_pages=4, page_tokens=16)                        # 64 tokens in all
    s = Scheduler(ex, SchedulerOptions(max_batch=4, prefill_token_budget=64))
    s.submit(Request("big", list(range(40)), greedy(9)))                # 48 positions: 3 pages
    s.submit(Request("next", list(range(20)), greedy(5)))               # 24 positions: 2 pages
    s.submit(Request("small", [1, 2], greedy(2)))                       # 1 page: would fit now
    info = s.step()
    assert info.admitted == 1 and info.pending == 2                     # small did not overtake next
    seen_waiting = 0
    while any(l.request.id == "big" for l in s.active + list(s.prefilling)):
        info = s.step()
        ids = {r for r, _, _ in ex.steps[-1]}
        if "next" not in ids:
            seen_waiting += 1
        assert ex.cache.reserved_pages(0) <= 4
    assert seen_waiting >= 7                                            # it waited while big decoded
    done = {c.id: c for c in s.run_to_completion()}
    assert sorted(done) == ["next", "small"] or sorted(done) == ["big", "next", "small"]
    assert ex.cache.free_pages(0) == 4 and ex.cache.reserved_pages(0) == 0


def test_requests_that_can_never_run_are_refused_at_submit():
    ex = FakeExecutor(n_pages=4, page_tokens=16)
    s = Scheduler(ex)
    with pytest.raises(SchedulerError, match="KV pages"):
        s.submit(Request("x", list(range(60)), greedy(10)))             # 69 positions > 64
    with pytest.raises(SchedulerError, match="cache positions"):
        s.submit(Request("y", list(range(500)), greedy(20)))            # beyond the context
    with pytest.raises(SchedulerError, match="positive"):
        s.submit(Request("z", [], greedy(1)))
    with pytest.raises(SchedulerError, match="vocabulary"):
        s.submit(Request("v", [1, 1000], greedy(1)))
    with pytest.raises(ValueError, match="temperature"):
        s.submit(Request("t", [1], SamplingParams(temperature=float("nan"))))
    s.submit(Request("ok", [1, 2, 3], greedy(1)))
    with pytest.raises(SchedulerError, match="already queued"):
        s.submit(Request("ok", [4], greedy(1)))
    assert not ex.cache.live_requests()                                 # nothing owned pages yet


def test_max_batch_bounds_the_residents_and_slots_are_reused():
    ex = FakeExecutor(n_pages=64, max_requests=2)
    s = Scheduler(ex, SchedulerOptions(max_batch=2, prefill_token_budget=64))
    for i in range(5):
        s.submit(Request(i, [1, 2, 3], greedy(2)))
    most = 0
    while s.has_work():
        s.step()
        most = max(most, len(s.active) + len(s.prefilling))
    assert most == 2 and len(s.done) == 5
    assert [c.id for c in s.done] == [0, 1, 2, 3, 4]


def test_first_token_comes_from_the_last_prompt_row_and_eos_stops():
    ex = FakeExecutor(n_pages=64)
    s = Scheduler(ex)
    s.submit(Request("a", [5, 6, 7], SamplingParams(max_tokens=50, eos_token_id=(2 * 7 + 7) % 1000)))
    info = s.step()
    assert ex.steps[0] == [("a", 3, [2])] and info.first_tokens == 1 and info.finished == 1
    assert s.done[0].tokens == [21] and s.done[0].finish_reason == "eos"


def test_greedy_requests_draw_nothing_and_sampled_ones_get_their_own_generator():
    ex = FakeExecutor(n_pages=64)
    seen = []
    ex.sample = lambda logits, rows: [seen.append([(p.is_greedy, None if r is None else r.state)
                                                   for p, r in rows]) or 1 for _ in rows][:len(rows)]
    s = Scheduler(ex)
    s.submit(Request("g", [1, 2], greedy(2)))
    s.submit(Request("t", [1, 2], SamplingParams(max_tokens=2, temperature=0.8, seed=42)))
    s.run_to_completion()
    assert seen[0][0] == (True, None)
    assert seen[0][1] == (False, 42 | 1)


def test_cancel_gives_everything_back_in_every_state():
    ex = FakeExecutor(n_pages=8)
    s = Scheduler(ex, SchedulerOptions(max_batch=2, prefill_token_budget=16))
    s.submit(Request("a", list(range(30)), greedy(4)))
    s.submit(Request("b", list(range(10)), greedy(4)))
    s.submit(Request("c", list(range(10)), greedy(4)))
    s.step()
    assert s.cancel("c") and s.cancel("a")                 # pending and prefilling
    s.step(); s.step()
    assert s.cancel("b") and not s.cancel("nobody")        # active
    assert ex.cache.free_pages(0) == 8 and ex.cache.reserved_pages(0) == 0
    assert {c.id: c.finish_reason for c in s.done} == {"a": "cancelled", "b": "cancelled",
                                                        "c": "cancelled"}
    assert not s.has_work()


class LaggedExecutor(FakeExecutor):
    """An executor that keeps the latest token of each request 'on the device' and
    hands the values over one call later, like the engine's `sample_deferred`."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.device_tokens = {}
        self.reads = 0

    def step(self, entries):
        from crucible_b200.engine import DEVICE_TOKEN
        fixed = []
        for e in entries:
            tokens = list(e.tokens)
            if tokens == [DEVICE_TOKEN]:
                tokens = [self.device_tokens[e.request]]
            fixed.append(type(e)(e.request, tokens, e.want))
        return super().step(fixed)

    def sample_deferred(self, logits, rows, requests):
        ids = FakeExecutor.sample(self, logits, rows)
        for r, tok in zip(requests, ids):
            self.device_tokens[r] = tok
        outer = self

        class Pending:
            def get(self_inner):
                outer.reads += 1
                return ids
        return Pending()


def test_token_values_may_lag_one_step_without_changing_the_result():
    prompts = {"a": list(range(50)), "b": list(range(20)), "c": [7, 8, 9]}

    def run(executor):
        s = Scheduler(executor, SchedulerOptions(max_batch=4, prefill_token_budget=32))
        for name, prompt in prompts.items():
            s.submit(Request(name, prompt, greedy(5 if name != "c" else 1)))
        return {c.id: c.tokens for c in s.run_to_completion()}, executor.steps

    want, steps_sync = run(FakeExecutor(n_pages=64))
    lagged = LaggedExecutor(n_pages=64)
    got, steps_lagged = run(lagged)
    assert got == want and all(len(v) == (1 if k == "c" else 5) for k, v in got.items())
    shape = lambda steps: [[(r, n) for r, n, _ in step] for step in steps]
    assert shape(steps_lagged) == shape(steps_sync)
    assert lagged.cache.free_pages(0) == 64 and lagged.reads > 0
    # a request that stops on a token value is run with its values at hand
    s = Scheduler(LaggedExecutor(n_pages=64))
    s.submit(Request("e", [5, 6, 7], SamplingParams(max_tokens=50, eos_token_id=(2 * 7 + 7) % 1000)))
    assert [c.finish_reason for c in s.run_to_completion()] == ["eos"]


class ChoosingExecutor(LaggedExecutor):
    """An executor whose step can choose its tokens itself, like the engine's `step_choosing`."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.chosen_steps = 0

    def step_choosing(self, entries):
        assert all(list(e.want) == [len(e.tokens) - 1] for e in entries)
        self.chosen_steps += 1
        logits = self.step(entries)
        rows = [(greedy(1), None)] * len(entries)
        return logits, self.sample_deferred(logits, rows, [e.request for e in entries])


def test_steps_whose_rows_are_all_greedy_choose_for_themselves():
    """Every entry of the step chooses a token, greedily, and no request can end on a token's
    value: the scheduler hands the choice to the step; a step with an unfinished portion, a
    sampled row or an end-of-sequence token goes the usual way.  The tokens are the same."""
    prompts = {"a": list(range(50)), "b": list(range(20)), "c": [7, 8, 9]}

    def run(executor, sampled=False):
        s = Scheduler(executor, SchedulerOptions(max_batch=4, prefill_token_budget=32))
        for name, prompt in prompts.items():
            params = greedy(5)
            if sampled and name == "c":
                params = SamplingParams(max_tokens=5, temperature=0.7, top_k=3, seed=1)
            s.submit(Request(name, prompt, params))
        return {c.id: c.tokens for c in s.run_to_completion()}, executor.steps

    want, steps_sync = run(FakeExecutor(n_pages=64))
    choosing = ChoosingExecutor(n_pages=64)
    got, steps = run(choosing)
    assert got == want
    portions = sum(1 for step in steps if any(not w for _, _, w in step))      # steps with an unfinished portion
    assert choosing.chosen_steps == len(steps) - portions > 0
    # one sampled request: its steps are not handed over
    mixed = ChoosingExecutor(n_pages=64)
    got_mixed, steps_mixed = run(mixed, sampled=True)
    assert got_mixed["a"] == want["a"] and got_mixed["b"] == want["b"]
    assert 0 < mixed.chosen_steps < len(steps_mixed) - sum(1 for st in steps_mixed if any(not w for _, _, w in st))


def test_an_executor_that_fails_mid_run_leaves_nothing_behind():
    """The executor raises in the middle of a run (the reference injects a device
    failure the same way, `engine/src/server.rs:1187-1227`): every live request's
    pages, reservation and state slot are returned, and the queue is empty."""
    class Failing(FakeExecutor):
        def step(self, entries):
            if len(self.steps) == 3:
                raise RuntimeError("injected device failure")
            return super().step(entries)

    ex = Failing(n_pages=32, max_requests=3)
    s = Scheduler(ex, SchedulerOptions(max_batch=3, prefill_token_budget=24))
    for i, n in enumerate([40, 10, 30, 12]):
        s.submit(Request(f"r{i}", list(range(n)), greedy(6)))
    with pytest.raises(RuntimeError, match="injected"):
        s.run_to_completion()
    assert len(ex.steps) == 3
    assert not ex.cache.live_requests()
    assert ex.cache.free_pages(0) == 32 and ex.cache.reserved_pages(0) == 0
    assert ex.cache.slots.free_slots == 3
    assert not s.has_work() and not s.pending
    ex.cache.check_invariants()
    # the same executor serves a new run afterwards
    ex.steps.append("recovered")
    s2 = Scheduler(ex, SchedulerOptions(max_batch=3, prefill_token_budget=24))
    s2.submit(Request("again", list(range(9)), greedy(3)))
    assert len(s2.run_to_completion()[0].tokens) == 3
