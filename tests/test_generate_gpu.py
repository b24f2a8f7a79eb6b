"""Generation through the Python entry point and the scheduler, long decoding,
and the first tokens of a sequence, against the plain implementation."""
import subprocess
import sys
import os

import numpy as np
import pytest
import torch

import helpers
import plain_model as pm
from helpers import TINY, TOLERANCE, Trace

pytestmark = pytest.mark.gpu


def _llm(folder, dtype, name, **kw):
    from crucible_b200 import LLM
    return LLM(folder, dtype=dtype, page_tokens=TINY[name]["page_tokens"], **kw)


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_greedy_generation_float32_is_token_identical(tmp_path, name):
    from crucible_b200 import SamplingParams
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    lengths = [7, 33, 64] if name == "tiny-a" else [1, 17, 50, 95, 130]
    prompts = [helpers.random_tokens(vocab, n, 40 + i) for i, n in enumerate(lengths)]
    n_new = 16 if name == "tiny-a" else 24
    cfg, w = pm.read_folder(folder)
    want = [pm.plain_generate(cfg, w, p, n_new) for p in prompts]
    # prompts chunked at 24 tokens and mixed with decodes, few pages, graphs on
    llm = _llm(folder, "float32", name, max_batch=3, prefill_token_budget=24,
               kv_pages=3 * (-(-(max(lengths) + n_new) // TINY[name]["page_tokens"])))
    got = llm.generate(prompts, SamplingParams(max_tokens=n_new))
    assert got == want
    assert any(s.prefill_tokens and s.decoded for s in llm.last_steps), "no mixed step happened"
    assert not llm.engine._graph_failed
    assert llm.engine._graph_replays > 0
    if name == "tiny-b":
        # portions of 24 tokens beside the same number of decoding requests come again and
        # again: such a step is captured at its second occurrence and replayed after that
        assert llm.engine._prompt_graph_replays > 0, "no step with a prompt portion was replayed"
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.live_requests()
    # the same without graphs and in one piece
    llm2 = _llm(folder, "float32", name, max_batch=8, prefill_token_budget=1024, graph=False)
    assert llm2.generate(prompts, SamplingParams(max_tokens=n_new)) == want


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_greedy_generation_bfloat16_follows_the_plain_model(tmp_path, name):
    """bfloat16 rounds, so a token may differ where the two best logits are
    close; every token must be the plain model's choice or within the rounding
    band of it, given the engine's own prefix."""
    from crucible_b200 import SamplingParams
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 60 + i) for i, n in enumerate([5, 40, 90])]
    llm = _llm(folder, "bfloat16", name, max_batch=4, prefill_token_budget=32)
    got = llm.generate(prompts, SamplingParams(max_tokens=20))
    cfg, w = pm.read_folder(folder)
    exact = 0
    for prompt, out in zip(prompts, got):
        assert len(out) == 20
        seq = list(prompt)
        for tok in out:
            logits = pm.plain_forward(cfg, w, seq)[-1]
            best = int(logits.argmax())
            band = TOLERANCE["bfloat16"] * float(logits.abs().max())
            assert float(logits[best] - logits[tok]) <= 2 * band, "token outside the rounding band"
            exact += int(tok == best)
            seq.append(tok)
    assert exact >= 0.9 * 60


def test_seeded_temperature_sampling_matches_the_plain_sampler(tmp_path):
    from crucible_b200 import SamplingParams
    name = "tiny-b"
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 80 + i) for i, n in enumerate([1, 17, 50])]
    params = [SamplingParams(max_tokens=24, temperature=0.8, top_k=40, seed=1234 + i)
              for i in range(3)]
    cfg, w = pm.read_folder(folder)
    want = [pm.plain_generate(cfg, w, p, 24, 0.8, 40, 1234 + i) for i, p in enumerate(prompts)]
    llm = _llm(folder, "float32", name, max_batch=4, prefill_token_budget=24)
    got = llm.generate(prompts, params)
    assert got == want
    # a request's sampled sequence does not depend on its neighbours
    alone = _llm(folder, "float32", name, max_batch=1).generate([prompts[1]], params[1])
    assert alone[0] == want[1]
    # greedy and sampled requests side by side
    mixed = llm.generate(prompts[:2], [SamplingParams(max_tokens=8), params[1]])
    assert mixed[0] == pm.plain_generate(cfg, w, prompts[0], 8) and mixed[1] == want[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_long_decoding_and_first_tokens(tmp_path, name, dtype):
    """A 3-token prompt, then 300 tokens one by one (crossing many pages and, in
    the split attention, a chunk edge); logits wanted from the very first token."""
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    tokens = helpers.random_tokens(vocab, 303, 11)
    trace = Trace()
    trace.step([("a", tokens[:1], [0])])
    trace.step([("a", tokens[1:3], [0, 1])])
    for i in range(3, len(tokens)):
        trace.step([("a", [tokens[i]], [0])], end=["a"] if i == len(tokens) - 1 else [])
    out = str(tmp_path / "out")
    helpers.replay_in_process(folder, dtype, trace, out, 320, TINY[name]["page_tokens"])
    got = helpers.collect(trace, out, vocab)
    ref = helpers.plain_logits(folder, tokens)
    for pos in range(len(tokens)):
        err = helpers.relative_error(got[("a", pos)], ref[pos])
        assert err <= TOLERANCE[dtype], f"position {pos}: relative error {err:.3g}"


def test_peaky_attention_over_many_pages(tmp_path):
    """With random weights attention is nearly uniform and a lost key hides in
    the average.  Here the query and key projections are scaled by 3 (scores by
    9), so single keys carry much of the weight and an engine that loses one (a
    page's edge, a chunk's edge) is off by far more than rounding.  The factor is
    kept where the plain implementation's own float32 rounding noise (3e-6 of the
    largest logit, measured against float64) stays well under the tolerance."""
    from crucible_b200.weights import SafetensorsFile, write_safetensors
    name = "tiny-a"
    folder = helpers.make_folder(tmp_path, name)
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.get(n) for n in f.names()}
    f.close()
    for n in tensors:
        if "q_proj" in n or "k_proj" in n:
            tensors[n] = (tensors[n].float() * 3.0).bfloat16()
    write_safetensors(path, tensors)
    vocab = TINY[name]["config"]["vocab_size"]
    tokens = helpers.random_tokens(vocab, 400, 21)
    ref = helpers.plain_logits(folder, tokens)

    def decoded(dtype):
        trace = Trace()
        trace.step([("a", tokens[:270], [269])])
        for i in range(270, 400):
            trace.step([("a", [tokens[i]], [0])], end=["a"] if i == 399 else [])
        out = str(tmp_path / f"out-{dtype}")
        helpers.replay_in_process(folder, dtype, trace, out, 448, 16)
        return helpers.collect(trace, out, vocab)

    got = decoded("float32")
    worst = max(helpers.relative_error(got[k], ref[k[1]]) for k in got)
    assert worst <= TOLERANCE["float32"], worst
    # bfloat16 rounds the queries and keys themselves and the scaling multiplies that
    # rounding in the scores, so for bfloat16 the factor is 1.5 (scores by 2.25): still
    # far from uniform attention, with the rounding noise inside the usual tolerance.
    for n in tensors:
        if "q_proj" in n or "k_proj" in n:
            tensors[n] = (tensors[n].float() * 0.5).bfloat16()
    write_safetensors(path, tensors)
    ref = helpers.plain_logits(folder, tokens)
    got = decoded("bfloat16")
    worst = max(helpers.relative_error(got[k], ref[k[1]]) for k in got)
    assert worst <= TOLERANCE["bfloat16"], worst


def test_command_line_generate(tmp_path):
    name = "tiny-a"
    folder = helpers.make_folder(tmp_path, name)
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "llm-engine"), "generate",
                           folder, "--prompt-ids", "5,17,3,200", "--max-tokens", "6",
                           "--temperature", "0", "--dtype", "float32", "--gpu", "--graph"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    import json
    out = json.loads(proc.stdout.strip().splitlines()[0])
    cfg, w = pm.read_folder(folder)
    assert out["tokens"] == pm.plain_generate(cfg, w, [5, 17, 3, 200], 6)
    assert "decode:" in proc.stderr and "prefill:" in proc.stderr


def test_step_refuses_malformed_batches(tmp_path):
    from crucible_b200.engine import Engine, EngineOptions, StepEntry, StepError
    from crucible_b200.cache import PoolExhausted
    folder = helpers.make_folder(tmp_path, "tiny-a")
    eng = Engine(folder, EngineOptions(dtype="float32", n_pages=4, max_requests=2))
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([StepEntry("a", [1, 256], [0])])
    with pytest.raises(StepError, match="twice"):
        eng.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(StepError, match="no tokens"):
        eng.step([StepEntry("a", [], [])])
    eng.step([StepEntry("a", list(range(40)), [39])])
    with pytest.raises(PoolExhausted):
        eng.step([StepEntry("b", list(range(30)), [])])       # 3 + 2 pages > 4
    assert not eng.has_request("b") or eng.held_tokens("b") == 0
    assert eng.held_tokens("a") == 40
    eng.cache.check_invariants()
    eng.finish("a")
    assert eng.cache.free_pages(0) == 4


# ---------------------------------------------------------------------------
# failure paths, made to happen without faulting, trapping or hanging anything
# ---------------------------------------------------------------------------

def test_a_wait_that_runs_out_is_reported_and_the_engine_recovers(tmp_path):
    """A kernel waits, bounded by a short limit, on a barrier at which nothing arrives,
    and records its give-up code in the status word as the tensor-core kernels do.  The
    product reads the word where the host waits anyway: generation raises instead of
    returning tokens chosen from a step that is not valid, gives back everything the
    run held, and the next run is clean."""
    from crucible_b200 import SamplingParams
    from crucible_b200.ops import tensor_core
    name = "tiny-c"
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 70 + i) for i, n in enumerate([80, 9])]
    llm = _llm(folder, "bfloat16", name, max_batch=2)
    want = llm.generate(prompts, SamplingParams(max_tokens=6))
    tensor_core.check_status(llm.engine.device)                 # nothing gave up so far
    failures = tensor_core.FAILURES[0]

    tensor_core.run_wait_probe(llm.engine.device, limit=2048)   # returns after 2,048 polls
    with pytest.raises(tensor_core.KernelGaveUp, match="status 4"):
        llm.generate(prompts, SamplingParams(max_tokens=6))
    assert tensor_core.FAILURES[0] == failures + 1
    assert not llm.engine.cache.live_requests()
    llm.engine.cache.check_invariants()
    assert int(tensor_core.status_word(llm.engine.device).item()) == 0
    assert llm.generate(prompts, SamplingParams(max_tokens=6)) == want

    # the trace replayer reads the word too, before it writes a step's logits
    tokens = prompts[0]
    trace = Trace()
    trace.step([("a", tokens, [len(tokens) - 1])], end=["a"])
    from crucible_b200.engine import replay
    import io
    engine = replay.make_engine(folder, "bfloat16", 128, TINY[name]["page_tokens"])
    tensor_core.run_wait_probe(engine.device, limit=2048)
    out = tmp_path / "replay-out"
    with pytest.raises(tensor_core.KernelGaveUp):
        replay.run(engine, io.StringIO(trace.text()), str(out), io.StringIO())
    assert not (out / "0.f32").exists()
    tensor_core.check_status(engine.device)                     # cleared


def test_a_capture_that_fails_leaves_the_engine_eager_and_right(tmp_path, monkeypatch):
    """`torch.cuda.graph` is made to raise when a step is captured (as
    `engine/src/gpu_model.rs:3199-3222` remembers a failed capture): the engine notes it,
    runs every further step eagerly, leaves no capture open, and the tokens are the same."""
    import torch
    from crucible_b200 import SamplingParams
    name = "tiny-a"
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 30 + i) for i, n in enumerate([12, 30])]
    want = _llm(folder, "float32", name, max_batch=2, graph=False).generate(
        prompts, SamplingParams(max_tokens=10))

    class Refusing:
        def __init__(self, *a, **k):
            raise RuntimeError("capture refused (injected)")

    llm = _llm(folder, "float32", name, max_batch=2)
    monkeypatch.setattr(torch.cuda, "graph", Refusing)
    got = llm.generate(prompts, SamplingParams(max_tokens=10))
    assert got == want
    assert llm.engine._graph_failed and "injected" in llm.engine._graph_error
    assert not llm.engine._graphs
    assert not torch.cuda.is_current_stream_capturing()
    monkeypatch.undo()
    assert llm.generate(prompts, SamplingParams(max_tokens=10)) == want      # still eager, still right
    assert llm.engine._graph_replays == 0


def test_step_refuses_a_page_named_by_two_requests(tmp_path):
    """An allocator that hands out a page that is still held (made to happen here by
    putting a held page back on the free stack): the step that would upload the second
    request's table is refused before anything is written, and changes nothing."""
    from crucible_b200.engine import Engine, EngineOptions, StepEntry, StepError
    folder = helpers.make_folder(tmp_path, "tiny-a")
    eng = Engine(folder, EngineOptions(dtype="float32", n_pages=8, max_requests=3))
    tokens = helpers.random_tokens(256, 40, 1)
    before = eng.step([StepEntry("a", tokens[:20], [19])]).clone()
    held = eng.cache.block_table("a", 0)[0]
    pool = eng.cache.pools[0]
    free_before = pool.free_pages
    pool.release(held)                            # the fault: a held page looks free
    with pytest.raises(StepError, match="another live request"):
        eng.step([StepEntry("b", tokens[:5], [4])])
    assert not eng.has_request("b")
    # rolled back to where the fault left it: the same page is the next one handed out
    assert pool.free_pages == free_before + 1 and not pool.is_in_use(held)
    assert pool.alloc() == held                   # undo the fault
    eng.cache.check_invariants()
    # request a is untouched: the same logits as a run that never saw the fault
    again = Engine(folder, EngineOptions(dtype="float32", n_pages=8, max_requests=3))
    again.step([StepEntry("a", tokens[:20], [19])])
    got = eng.step([StepEntry("a", tokens[20:], [19])])
    want = again.step([StepEntry("a", tokens[20:], [19])])
    assert torch.equal(got, want) and torch.equal(before, before)
    # a table entry changed behind the engine's back is found by the full check
    eng.step([StepEntry("c", tokens[:5], [])])
    eng.cache._poke("c", 0, 0, eng.cache.block_table("a", 0)[1])
    with pytest.raises(StepError, match="another live request"):
        eng.check_tables()


def test_device_token_needs_a_deferred_sample(tmp_path):
    """`DEVICE_TOKEN` stands for the token the engine last chose for the request and kept
    on the device; a request that never had one chosen that way (a new one in a slot
    whose last owner had) is refused instead of reading the old owner's token."""
    from crucible_b200 import SamplingParams
    from crucible_b200.engine import DEVICE_TOKEN, Engine, EngineOptions, StepEntry, StepError
    folder = helpers.make_folder(tmp_path, "tiny-a")
    eng = Engine(folder, EngineOptions(dtype="float32", n_pages=8, max_requests=1))
    logits = eng.step([StepEntry("a", [5, 6, 7], [2])])
    with pytest.raises(StepError, match="no token on the device"):
        eng.step([StepEntry("a", [DEVICE_TOKEN], [0])])
    ids = eng.sample_deferred(logits, [(SamplingParams(), None)], ["a"])
    eng.step([StepEntry("a", [DEVICE_TOKEN], [0])])          # now it has one
    assert 0 <= ids.get()[0] < 256
    eng.finish("a")
    eng.step([StepEntry("b", [1, 2], [1])])                  # takes the same slot
    with pytest.raises(StepError, match="no token on the device"):
        eng.step([StepEntry("b", [DEVICE_TOKEN], [0])])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_choosing_step_chooses_what_its_logits_say(tmp_path, dtype):
    """`step_choosing`: the greedy choice is part of the step (captured with it once the
    step replays a graph).  The ids are the argmax of the step's own logits, they are what
    `DEVICE_TOKEN` feeds into the next step (an engine fed the same ids explicitly gives the
    same logits), and a replayed step writes the slots of the requests it is run for, not of
    those it was captured with."""
    from crucible_b200.engine import DEVICE_TOKEN, Engine, EngineOptions, StepEntry, StepError
    folder = helpers.make_folder(tmp_path, "tiny-b")
    eng = Engine(folder, EngineOptions(dtype=dtype, n_pages=40, max_requests=4))
    ref = Engine(folder, EngineOptions(dtype=dtype, n_pages=40, max_requests=4))
    vocab = eng.config.vocab_size
    prompts = {r: helpers.random_tokens(vocab, 9 + 4 * i, 20 + i) for i, r in enumerate("abc")}
    with pytest.raises(StepError, match="last token"):
        eng.step_choosing([StepEntry("a", prompts["a"], [0])])

    def both(names, tokens_of):
        logits, pending = eng.step_choosing([StepEntry(r, tokens_of[r], [len(tokens_of[r]) - 1]) for r in names])
        ids = pending.get()
        assert ids == logits.argmax(dim=-1).tolist()
        return logits.clone(), ids

    want = ref.step([StepEntry(r, prompts[r], [len(prompts[r]) - 1]) for r in "abc"]).clone()
    logits, ids = both("abc", prompts)
    assert torch.equal(logits, want)
    fed = dict(zip("abc", ids))
    for step in range(8):                                   # the later ones replay their graphs
        want = ref.step([StepEntry(r, [fed[r]], [0]) for r in "abc"]).clone()
        logits, ids = both("abc", {r: [DEVICE_TOKEN] for r in "abc"})
        assert torch.equal(logits, want), step
        fed = dict(zip("abc", ids))
    assert eng._graphs and not eng._graph_failed, eng._graph_error
    # another set of requests in other slots, the same shape of step
    eng.finish("a")
    prompts["d"] = helpers.random_tokens(vocab, 7, 31)
    _, first = both("d", prompts)
    names = "bdc"                                           # other slots in other rows than it was captured with
    fed["d"] = first[0]
    ref.finish("a")
    ref.step([StepEntry("d", prompts["d"], [])])
    for step in range(4):
        want = ref.step([StepEntry(r, [fed[r]], [0]) for r in names]).clone()
        logits, ids = both(names, {r: [DEVICE_TOKEN] for r in names})
        assert torch.equal(logits, want), step
        fed = dict(zip(names, ids))
    eng.cache.check_invariants()


def test_eos_and_cancel_through_the_engine(tmp_path):
    """`eos_token_id` ends a request at the token the plain model also chooses, and a
    request cancelled between steps gives back its pages while the others go on."""
    from crucible_b200 import SamplingParams
    from crucible_b200.engine.scheduler import Request, Scheduler, SchedulerOptions
    name = "tiny-a"
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 90 + i) for i, n in enumerate([9, 30, 21])]
    cfg, w = pm.read_folder(folder)
    full = [pm.plain_generate(cfg, w, p, 14) for p in prompts]
    llm = _llm(folder, "float32", name, max_batch=3, prefill_token_budget=16)
    # the fifth token of request 0 is made its end-of-sequence token
    eos = full[0][4]
    cut = full[0].index(eos) + 1
    params = [SamplingParams(max_tokens=14, eos_token_id=eos), SamplingParams(max_tokens=14),
              SamplingParams(max_tokens=14)]
    got = llm.generate(prompts, params)
    assert got[0] == full[0][:cut] and got[0][-1] == eos
    assert got[1] == full[1] and got[2] == full[2]
    assert not llm.engine.cache.live_requests()
    # cancel: request 1 is taken out after a few steps; the others are not disturbed
    sched = Scheduler(llm.engine, SchedulerOptions(max_batch=3, prefill_token_budget=16))
    for i, p in enumerate(prompts):
        sched.submit(Request(i, p, SamplingParams(max_tokens=14)))
    for _ in range(5):
        sched.step()
    free_before = llm.engine.cache.free_pages(0)
    assert sched.cancel(1)
    assert llm.engine.cache.free_pages(0) > free_before and not llm.engine.has_request(1)
    done = {c.id: c for c in sched.run_to_completion()}
    assert done[1].finish_reason == "cancelled" and done[1].tokens == full[1][:len(done[1].tokens)]
    assert done[0].tokens == full[0] and done[2].tokens == full[2]
    assert done[0].finish_reason == "length"
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.live_requests()


def test_stage_table_attributes_a_step_to_the_parts(tmp_path):
    """The opt-in stage table: with `profile=True` every part is timed with CUDA events,
    steps run eagerly, the tokens are the same, and the stages are the model's parts."""
    from crucible_b200 import SamplingParams
    name = "tiny-b"
    folder = helpers.make_folder(tmp_path, name)
    vocab = TINY[name]["config"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 20 + i) for i, n in enumerate([40, 9])]
    plain = _llm(folder, "float32", name, max_batch=2)
    assert plain.engine.profiler is None
    want = plain.generate(prompts, SamplingParams(max_tokens=6))
    llm = _llm(folder, "float32", name, max_batch=2, profile=True)
    assert llm.generate(prompts, SamplingParams(max_tokens=6)) == want
    assert llm.engine._graph_replays == 0 and not llm.engine._graphs
    rows = {r["stage"]: r for r in llm.engine.profiler.table()}
    layers = TINY[name]["config"]["num_hidden_layers"]
    steps = llm.engine.profiler.steps
    assert steps == len(llm.last_steps) > 5
    assert rows["layer.mixer[attention]"]["calls"] == steps * layers
    assert rows["layer.feed_forward[swiglu]"]["calls"] == steps * layers
    assert rows["layer.mixer_norm"]["calls"] == steps * layers
    assert rows["embedding"]["calls"] == steps and rows["head"]["calls"] == steps
    assert all(r["ms"] > 0 for r in rows.values())
    assert abs(sum(r["share"] for r in rows.values()) - 1.0) < 1e-2
    assert "layer.mixer[attention]" in llm.engine.profiler.text()
