"""Trace replay on the GPU against the plain implementation, in float32 and in
bfloat16: each request alone and whole; most of it in one step and the last 32
tokens one by one; in portions of changing size down to two tokens; and mixed,
up to four live requests, portions of some beside decoded tokens of others,
with so few pages that they are used again."""
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
from helpers import TINY, TOLERANCE, Trace

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny-a": [7, 33, 64, 150], "tiny-b": [1, 17, 50, 95, 130], "tiny-c": [70, 150, 201]}


def _one_at_a_time(name):
    """--max-tokens when one request is live at a time: the longest, rounded up to 64."""
    return max(192, -(-max(LENGTHS[name]) // 64) * 64)


def _vocab(name):
    return TINY[name]["config"]["vocab_size"]


def _requests(name):
    return {f"r{i}": helpers.random_tokens(_vocab(name), n, 100 + i)
            for i, n in enumerate(LENGTHS[name])}


def _check(name, dtype, model_dir, trace, out_dir, requests, max_tokens):
    helpers.replay_in_process(model_dir, dtype, trace, out_dir, max_tokens,
                              TINY[name]["page_tokens"])
    got = helpers.collect(trace, out_dir, _vocab(name))
    assert got, "the trace asked for nothing"
    worst = 0.0
    for rid, tokens in requests.items():
        ref = helpers.plain_logits(model_dir, tokens)
        keys = sorted(k for k in got if k[0] == rid)
        assert keys, f"no logits for {rid}"
        mine = np.stack([got[k] for k in keys])
        theirs = np.stack([ref[k[1]] for k in keys])
        err = helpers.relative_error(mine, theirs)
        if err > TOLERANCE[dtype]:
            # name the first wrong place: what is special about it?
            for k in keys:
                e = helpers.relative_error(got[k], ref[k[1]])
                if e > TOLERANCE[dtype]:
                    pytest.fail(f"{name} {dtype}: request {rid} first differs at position "
                                f"{k[1]} (relative error {e:.3g}, allowed {TOLERANCE[dtype]})")
        worst = max(worst, err)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_each_request_alone_and_whole(tmp_path, name, dtype):
    model_dir = helpers.make_folder(tmp_path, name)
    requests = _requests(name)
    trace = Trace()
    for rid, tokens in requests.items():
        trace.step([(rid, tokens, list(range(len(tokens))))], end=[rid])
    _check(name, dtype, model_dir, trace, str(tmp_path / "out"), requests, _one_at_a_time(name))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_prompt_then_last_32_one_by_one(tmp_path, name, dtype):
    model_dir = helpers.make_folder(tmp_path, name)
    requests = {k: v for k, v in _requests(name).items() if len(v) > 40}
    trace = Trace()
    for rid, tokens in requests.items():
        head = len(tokens) - 32
        trace.step([(rid, tokens[:head], [head - 1])])
        for i in range(head, len(tokens)):
            trace.step([(rid, [tokens[i]], [0])], end=[rid] if i == len(tokens) - 1 else [])
    _check(name, dtype, model_dir, trace, str(tmp_path / "out"), requests, _one_at_a_time(name))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_portions_of_changing_size(tmp_path, name, dtype):
    model_dir = helpers.make_folder(tmp_path, name)
    requests = {k: v for k, v in _requests(name).items() if len(v) >= 33}
    sizes = [24, 7, 2, 13, 2, 31, 5, 17, 3, 40]
    trace = Trace()
    for rid, tokens in requests.items():
        at, i = 0, 0
        while at < len(tokens):
            n = min(sizes[i % len(sizes)], len(tokens) - at)
            if len(tokens) - at - n == 1:      # never leave a single token: portions go down to two
                n += 1
            last = at + n == len(tokens)
            trace.step([(rid, tokens[at:at + n], list(range(n)))], end=[rid] if last else [])
            at += n
            i += 1
    _check(name, dtype, model_dir, trace, str(tmp_path / "out"), requests, _one_at_a_time(name))


def _mixed_trace(requests, chunk, seed):
    """Up to four live requests; portions of prompts beside single tokens of
    requests that have reached their last 12 tokens ("decoding"); a request
    is sometimes left out of a step; finished requests free their pages for
    the ones still waiting."""
    import random
    rng = random.Random(seed)
    waiting = list(requests)
    live = {}
    trace = Trace()
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, ended = [], []
        for rid in list(live):
            tokens = requests[rid]
            at = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # sits this step out
            decode_from = max(1, len(tokens) - 12)
            if at >= decode_from:
                n = 1
            else:
                n = min(rng.choice([chunk, chunk // 2, 5, 2]), decode_from - at)
                if decode_from - at - n == 1 and n > 1:
                    n += 1 if at + n + 1 <= decode_from else 0
            want = list(range(n)) if n <= 2 or rng.random() < 0.5 else [n - 1]
            entries.append((rid, tokens[at:at + n], want))
            live[rid] = at + n
            if live[rid] == len(tokens):
                ended.append(rid)
        if entries:
            if rng.random() < 0.7:
                # as the scheduler orders a step: decoded tokens first, then portions (the
                # engine then runs the two kinds through different attention kernels)
                entries.sort(key=lambda e: len(e[1]) != 1)
            trace.step(entries, end=ended)
        for rid in ended:
            del live[rid]
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_mixed_requests_with_pages_used_again(tmp_path, name, dtype):
    model_dir = helpers.make_folder(tmp_path, name)
    base = _requests(name)
    # twice as many requests as fit at once, so that pages are used again
    requests = dict(base)
    for i, (rid, tokens) in enumerate(list(base.items())):
        requests[f"s{i}"] = helpers.random_tokens(_vocab(name), max(2, len(tokens) - 3), 500 + i)
    # tiny-c (two query heads to a KV head) gets portions of 48 tokens: 96 packed rows, so that
    # in bfloat16 its portions reach the tcgen05 tile kernel while other requests decode beside them
    trace = _mixed_trace(requests, 48 if name == "tiny-c" else 24, seed=7)
    # four live requests, each rounded up to a multiple of 64
    longest = sorted((-(-len(t) // 64) * 64 for t in requests.values()), reverse=True)
    max_tokens = sum(longest[:4])
    _check(name, dtype, model_dir, trace, str(tmp_path / "out"), requests, max_tokens)


def test_trace_run_program(tmp_path):
    """The program itself, as a user runs it: standard input, files, done lines."""
    name = "tiny-a"
    model_dir = helpers.make_folder(tmp_path, name)
    tokens = helpers.random_tokens(_vocab(name), 40, 9)
    trace = Trace()
    trace.step([("a", tokens[:30], [29])])
    trace.step([("a", tokens[30:], [0, 9])], end=["a"])
    out = str(tmp_path / "out")
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model",
                           model_dir, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                          input=trace.text(), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert proc.stdout.split() == ["done", "0", "done", "1"]
    got = helpers.collect(trace, out, _vocab(name))
    ref = helpers.plain_logits(model_dir, tokens)
    for (rid, pos), row in got.items():
        assert helpers.relative_error(row, ref[pos]) <= TOLERANCE["float32"]


# ---------------------------------------------------------------------------
# float32: the four ways of cutting give the same bits
# ---------------------------------------------------------------------------

def _wide_folder(tmp_path):
    """Two layers at the 120M shape's widths (768 wide, 12 query and 4 KV heads of 64,
    feed-forward 2,048) with a small vocabulary that is no power of two.  At this width
    a row of the residual stream is several float4 per lane and several warps per block,
    so two norm kernels that add in different orders give different bits; at the tiny
    widths they would agree by accident."""
    from crucible_b200.config import shape
    from crucible_b200.weights import write_random_model
    raw = shape("120m")
    raw.update(n_layer=2, vocab_size=1003, block_size=512)
    return write_random_model(raw, str(tmp_path / "wide"), seed=4, std=helpers.TEST_STD), 1003, 16


def _bit_equal_case(tmp_path, which):
    if which == "wide":
        return _wide_folder(tmp_path)
    return (helpers.make_folder(tmp_path, which), _vocab(which), TINY[which]["page_tokens"])


@pytest.mark.parametrize("which", ["wide", "tiny-b"])
def test_float32_cuts_are_bit_equal(tmp_path, which):
    """One request of more than 200 tokens run whole, token by token, in portions of
    changing size and mixed beside three other requests: in float32 every sum's order is
    a function of the problem alone (never of how many rows a step holds), so the logits
    at a position are the same bits in all four (the reference met the opposite three
    times: `README.md:2806-2814`, `docs/paged-attention-design.md:109-130`,
    `engine/kernels/kernels.cu:2100-2108`)."""
    model_dir, vocab, page = _bit_equal_case(tmp_path, which)
    n = 230
    main = helpers.random_tokens(vocab, n, 900)
    others = {f"o{i}": helpers.random_tokens(vocab, m, 910 + i) for i, m in enumerate([75, 140, 190])}
    places = list(range(0, n, 9)) + [n - 1]

    def collect_main(trace, sub):
        out = str(tmp_path / sub)
        helpers.replay_in_process(model_dir, "float32", trace, out, 4 * 256, page)
        got = helpers.collect(trace, out, vocab)
        return {pos: row for (rid, pos), row in got.items() if rid == "m"}

    whole = Trace()
    whole.step([("m", main, places)], end=["m"])
    one_by_one = Trace()
    for i, tok in enumerate(main):
        one_by_one.step([("m", [tok], [0] if i in places else [])], end=["m"] if i == n - 1 else [])
    portions = Trace()
    sizes, at, i = [24, 7, 2, 13, 2, 31, 5, 17, 3, 70, 40], 0, 0
    while at < n:
        m = min(sizes[i % len(sizes)], n - at)
        portions.step([("m", main[at:at + m], [p - at for p in places if at <= p < at + m])],
                      end=["m"] if at + m == n else [])
        at, i = at + m, i + 1
    # mixed: the main request in portions beside the others, which are fed in portions of
    # their own and then token by token; more than 64 rows in some steps, fewer in others
    mixed = Trace()
    fed = {rid: 0 for rid in others}
    at, i = 0, 0
    main_sizes = [40, 3, 66, 1, 1, 25, 90, 2, 1, 1]
    while at < n or any(fed[r] < len(t) for r, t in others.items()):
        entries, ended = [], []
        if at < n:
            m = min(main_sizes[i % len(main_sizes)], n - at)
            entries.append(("m", main[at:at + m], [p - at for p in places if at <= p < at + m]))
            at += m
            if at == n:
                ended.append("m")
        for j, (rid, toks) in enumerate(others.items()):
            if fed[rid] >= len(toks) or (i + j) % 4 == 3:
                continue
            m = 1 if fed[rid] >= len(toks) - 20 else min(30 + 7 * j, len(toks) - 20 - fed[rid])
            entries.append((rid, toks[fed[rid]:fed[rid] + m], [m - 1]))
            fed[rid] += m
            if fed[rid] == len(toks):
                ended.append(rid)
        if entries:
            mixed.step(entries, end=ended)
        i += 1

    ref = collect_main(whole, "whole")
    assert sorted(ref) == sorted(set(places))
    for name, trace in (("one by one", one_by_one), ("portions", portions), ("mixed", mixed)):
        got = collect_main(trace, name.replace(" ", "_"))
        assert sorted(got) == sorted(ref), name
        for pos in sorted(ref):
            assert np.array_equal(got[pos], ref[pos]), (
                f"{which}: {name} differs from the whole prompt at position {pos} "
                f"(largest difference {np.abs(got[pos] - ref[pos]).max():.3g})")
