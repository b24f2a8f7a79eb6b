"""The engine at the benchmark's layer sizes (two layers of the 120M shape): steps whose
shapes reach the kernels and rules that the tiny configurations cannot (256 x 256 tiles,
clusters that share K, the products' hand-over at 17 rows, replayed graphs of 64 rows).
The plain implementation would take minutes at this width, so the bfloat16 engine is
compared with the float32 engine, which the other tests hold against the plain
implementation, and the float32 engine with itself across ways of cutting."""
import random

import pytest
import torch

from helpers import TOLERANCE

pytestmark = pytest.mark.gpu


def _plan(vocab):
    rng = random.Random(3)
    long_prompt = [rng.randrange(vocab) for _ in range(2048)]
    others = {f"r{i}": [rng.randrange(vocab) for _ in range(40 + i)] for i in range(63)}
    plan = [[("a", long_prompt, [0, 2047])],                               # whole
            [("b", long_prompt[:1500], [])], [("b", long_prompt[1500:2000], [])],
            [("b", long_prompt[2000:2046], [])], [("b", long_prompt[2046:], [1])], "end b",
            # 63 short prompts beside a decoded token: thousands of rows in one step
            [("a", [7], [0])] + [(rid, toks, [len(toks) - 1]) for rid, toks in others.items()]]
    for _ in range(2):                                                     # 64 rows; the second replays
        plan.append([("a", [9], [0])] + [(rid, [11], [0]) for rid in others])
    for n in (24, 17, 8):                                                  # the products' hand-overs
        for _ in range(2):
            plan.append([("a", [5], [0])] + [(f"r{i}", [6], [0]) for i in range(n - 1)])
    return plan


def _run(folder, dtype, plan):
    from crucible_b200 import LLM
    from crucible_b200.engine import StepEntry
    from crucible_b200.ops import tensor_core
    llm = LLM(folder, dtype=dtype, max_batch=66, kv_pages=66 * 40 + 300, prefill_token_budget=4096)
    engine = llm.engine
    rows = []
    for step in plan:
        if step == "end b":
            engine.finish("b")
            continue
        logits = engine.step([StepEntry(rid, toks, want) for rid, toks, want in step])
        rows.extend(logits.float().cpu())
    tensor_core.check_status(engine.device)
    assert not engine._graph_failed
    engine.cache.check_invariants()
    return rows


def _config(which):
    from crucible_b200.config import shape
    if which == "120m":
        raw = shape("120m")
        raw["n_layer"] = 2
        return raw
    # the Llama spelling with heads of 128 and a long K: a quarter of the Llama-3-8B widths
    raw = shape("llama-8b")
    raw.update(num_hidden_layers=1, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2,
               intermediate_size=3584, vocab_size=32000, max_position_embeddings=4096)
    return raw


@pytest.mark.parametrize("which", ["120m", "heads-of-128"])
def test_bfloat16_follows_float32_at_the_benchmark_widths(tmp_path, which):
    from crucible_b200.weights import write_random_model
    raw = _config(which)
    folder = write_random_model(raw, str(tmp_path / "model"), seed=0)
    plan = _plan(raw["vocab_size"])
    ref = _run(folder, "float32", plan)
    got = _run(folder, "bfloat16", plan)
    assert len(ref) == len(got) > 200
    # the prompt whole and in portions: the same logits at its last position
    assert float((ref[1] - ref[2]).abs().max() / ref[1].abs().max()) < TOLERANCE["float32"]
    worst = max(float((r - g).abs().max() / r.abs().max()) for r, g in zip(ref, got))
    assert worst < TOLERANCE["bfloat16"], worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_benchmark_widths_against_the_plain_model(tmp_path, dtype):
    """Two layers of the 120M shape (768 wide, 12 / 4 heads of 64, feed-forward 2,048, the
    vocabulary of 50,304) against the plain implementation itself, not against another path
    of the engine: a prompt of 1,850 tokens in one step, which in bfloat16 reaches the
    256 x 256 product tiles, the product with the rotation in its epilogue and the tcgen05
    attention over 116 pages, then 40 tokens decoded one by one through the few-row products,
    the split attention and the 50,304-row head; logits wanted at 48 places."""
    import numpy as np
    import plain_model as pm
    from crucible_b200.engine import Engine, EngineOptions, StepEntry
    from crucible_b200.ops import tensor_core
    from crucible_b200.weights import write_random_model
    import helpers
    raw = _config("120m")
    folder = write_random_model(raw, str(tmp_path / "model"), seed=3, std=0.05)
    vocab = raw["vocab_size"]
    tokens = helpers.random_tokens(vocab, 1890, 77)
    prompt_places = [0, 1, 15, 16, 17, 255, 256, 511, 1023, 1024, 1848, 1849]
    places = prompt_places + list(range(1850, 1890))[:36]
    cfg, w = pm.read_folder(folder)
    ref = pm.plain_forward(cfg, w, tokens, rows=places).numpy()
    eng = Engine(folder, EngineOptions(dtype=dtype, page_tokens=16, n_pages=130, max_requests=2))
    got = [eng.step([StepEntry("a", tokens[:1850], prompt_places)]).float().cpu().numpy()]
    for i in range(1850, 1890):
        row = eng.step([StepEntry("a", [tokens[i]], [0])]).float().cpu().numpy()
        if i in places:
            got.append(row)
    tensor_core.check_status(eng.device)
    got = np.concatenate(got)
    assert got.shape == ref.shape == (48, vocab)
    assert eng._graph_replays > 30 and not eng._graph_failed, eng._graph_error
    for i, pos in enumerate(places):
        err = helpers.relative_error(got[i], ref[i])
        assert err <= TOLERANCE[dtype], f"position {pos}: relative error {err:.3g}"


def test_products_leave_the_next_norms_input_for_steps_of_many_rows(tmp_path):
    """A step of more than 16 rows: the output and down projections leave the next norm's
    input (all norms but a step's first and last then cost no launch), the q/k/v and gate/up
    products apply the rows' factors; the logits follow the float32 engine as they do with
    every norm a kernel of its own."""
    from crucible_b200 import ops
    from crucible_b200.engine import Engine, EngineOptions, StepEntry
    from crucible_b200.ops import tensor_core
    from crucible_b200.weights import write_random_model
    import helpers
    raw = _config("120m")
    folder = write_random_model(raw, str(tmp_path / "model"), seed=5, std=0.05)
    prompt = helpers.random_tokens(raw["vocab_size"], 333, 5)
    short = helpers.random_tokens(raw["vocab_size"], 40, 6)
    want = [0, 17, 332]

    def run(dtype, ahead):
        tensor_core.NORM_AHEAD = ahead
        try:
            eng = Engine(folder, EngineOptions(dtype=dtype, page_tokens=16, n_pages=120, max_requests=40))
            before = ops.LAUNCHES[0]
            rows = [eng.step([StepEntry("a", prompt, want)]).float().cpu()]
            launches = ops.LAUNCHES[0] - before
            # 24 decoded tokens of as many requests, twice (the second step replays its graph)
            rows.append(eng.step([StepEntry(f"r{i}", short, [39]) for i in range(24)]).float().cpu())
            for _ in range(2):
                rows.append(eng.step([StepEntry(f"r{i}", [7 + i], [0]) for i in range(24)]).float().cpu())
            tensor_core.check_status(eng.device)
            assert not eng._graph_failed
            return torch.cat(rows), launches
        finally:
            tensor_core.NORM_AHEAD = True
    ref, _ = run("float32", True)
    with_it, n_with = run("bfloat16", True)
    without, n_without = run("bfloat16", False)
    assert n_without - n_with == 2 * raw["n_layer"] - 1
    for got in (with_it, without):
        worst = float(((ref - got).abs().amax(1) / ref.abs().amax(1)).max())
        assert worst < helpers.TOLERANCE["bfloat16"], worst
