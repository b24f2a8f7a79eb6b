"""The native step packer (csrc/host_step.cpp) against a plain numpy packing of the same
step, and its checks.  Host code only: runs without a GPU."""
import ctypes
import random

import numpy as np
import pytest

from crucible_b200.engine.context import StepLayout
from crucible_b200.ops import build

DEVICE_TOKEN = -1


def _pack(counts, starts, slots, tokens, want_counts, wants, strides, rows, vocab=1000, max_context=4096):
    lib = build.load("host_step")
    n_req = len(counts)
    layout = StepLayout(sum(counts), n_req, sum(want_counts), tuple(strides))
    total = layout.offsets()["_total"][1]
    dst = np.full(total, -12345, dtype=np.int32)
    i32 = lambda x: np.asarray(x, dtype=np.int32)
    c, s_, sl, wc, w = i32(counts), i32(starts), i32(slots), i32(want_counts), i32(wants)
    t = np.asarray(tokens, dtype=np.int64)
    st = i32(strides)
    ptrs = (ctypes.c_void_p * max(1, len(rows)))(*[r.ctypes.data for r in rows])
    bad = ctypes.c_int32(-1)
    err = ctypes.create_string_buffer(256)
    fn = lib.cb_host_pack_step
    fn.restype = ctypes.c_int
    fn.argtypes = ([ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6
                   + [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                      ctypes.c_longlong, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int])
    code = fn(dst.ctypes.data, n_req, c.ctypes.data, s_.ctypes.data, sl.ctypes.data, t.ctypes.data,
              wc.ctypes.data, w.ctypes.data, len(strides), st.ctypes.data, ptrs, vocab, max_context,
              DEVICE_TOKEN, ctypes.byref(bad), err, 256)
    return code, bad.value, err.value.decode(), dst, layout


def _numpy_pack(counts, starts, slots, tokens, want_counts, wants, strides, rows):
    n_req = len(counts)
    layout = StepLayout(sum(counts), n_req, sum(want_counts), tuple(strides))
    off = layout.offsets()
    out = np.full(off["_total"][1], -12345, dtype=np.int32)

    def put(name, values):
        a, n = off[name]
        out[a:a + n] = values
    row_starts = np.concatenate([[0], np.cumsum(counts)])
    owner = np.repeat(np.arange(n_req), counts)
    ids = np.asarray(tokens, dtype=np.int64).copy()
    for r in range(n_req):
        if counts[r] == 1 and ids[row_starts[r]] == DEVICE_TOKEN:
            ids[row_starts[r]] = -(slots[r] + 1)
    put("token_ids", ids)
    put("positions", np.arange(sum(counts)) + (np.asarray(starts) - row_starts[:-1])[owner])
    put("row_request", owner)
    want_owner = np.repeat(np.arange(n_req), want_counts)
    put("logit_rows", row_starts[:-1][want_owner] + np.asarray(wants, dtype=np.int64))
    put("req_row_start", row_starts)
    put("req_context_len", np.asarray(starts) + np.asarray(counts))
    put("req_first_pos", starts)
    put("req_state_slot", slots)
    for g, stride in enumerate(strides):
        a, n = off[f"table{g}"]
        out[a:a + n] = np.concatenate([rows[g * n_req + r] for r in range(n_req)])
    return out


@pytest.mark.parametrize("seed", range(12))
def test_native_packing_equals_the_plain_one(seed):
    rng = random.Random(seed)
    n_req = rng.randint(1, 9)
    strides = [rng.choice([3, 8, 17]) for _ in range(rng.randint(1, 3))]
    counts = [rng.choice([1, 1, 1, 2, 5, 40]) for _ in range(n_req)]
    starts = [rng.randint(0, 500) for _ in range(n_req)]
    slots = rng.sample(range(16), n_req)
    tokens = []
    for n in counts:
        if n == 1 and rng.random() < 0.4:
            tokens.append(DEVICE_TOKEN)
        else:
            tokens += [rng.randrange(1000) for _ in range(n)]
    want = [sorted(rng.sample(range(n), rng.randint(0, min(n, 3)))) for n in counts]
    want_counts = [len(w) for w in want]
    wants = [p for w in want for p in w]
    rows = [np.asarray([rng.randrange(99) for _ in range(stride)], dtype=np.int32)
            for stride in strides for _ in range(n_req)]
    code, bad, err, got, layout = _pack(counts, starts, slots, tokens, want_counts, wants, strides, rows)
    assert code == 0, err
    ref = _numpy_pack(counts, starts, slots, tokens, want_counts, wants, strides, rows)
    # padding between pieces is never written; everything else is equal
    assert np.array_equal(got, ref)
    off = layout.offsets()
    assert all(a % 4 == 0 for a, _ in off.values())           # every piece on a 16-byte boundary


def test_native_offsets_follow_the_layout_rule():
    lib = build.load("host_step")
    for n_tokens, n_req, n_want, strides in ((1, 1, 1, (5,)), (2053, 7, 9, (129, 3)), (64, 64, 0, (256,))):
        off = StepLayout(n_tokens, n_req, n_want, strides).offsets()
        out = np.zeros(8 + len(strides) + 1, dtype=np.int32)
        st = np.asarray(strides, dtype=np.int32)
        lib.cb_host_step_offsets(n_tokens, n_req, n_want, len(strides), ctypes.c_void_p(st.ctypes.data),
                                 ctypes.c_void_p(out.ctypes.data))
        names = ["token_ids", "positions", "row_request", "logit_rows", "req_row_start", "req_context_len",
                 "req_first_pos", "req_state_slot"] + [f"table{g}" for g in range(len(strides))]
        assert [off[n][0] for n in names] == out[:-1].tolist()
        assert out[-1] == off["_total"][1]


def test_native_packer_refuses_bad_steps_and_names_the_request():
    row = [np.zeros(4, dtype=np.int32)] * 2
    base = dict(counts=[2, 1], starts=[0, 7], slots=[0, 1], tokens=[5, 6, 7], want_counts=[1, 1],
                wants=[1, 0], strides=[4], rows=row)
    assert _pack(**base)[0] == 0
    code, bad, err, *_ = _pack(**dict(base, tokens=[5, 1000, 7]))
    assert (code, bad) == (2, 0) and "vocabulary" in err
    code, bad, err, *_ = _pack(**dict(base, tokens=[5, 6, -2]))
    assert (code, bad) == (2, 1)
    code, bad, err, *_ = _pack(**dict(base, wants=[2, 0]))
    assert (code, bad) == (4, 0) and "wanted place" in err
    code, bad, err, *_ = _pack(**dict(base, want_counts=[2, 0], wants=[1, 1]))
    assert (code, bad) == (5, 0) and "ascend" in err
    code, bad, err, *_ = _pack(**dict(base, starts=[0, 4096]))
    assert (code, bad) == (3, 1) and "context" in err
    code, bad, err, *_ = _pack(**dict(base, counts=[2, 0], tokens=[5, 6], want_counts=[1, 0], wants=[1]))
    assert (code, bad) == (1, 1) and "no tokens" in err
    # a lone DEVICE_TOKEN stands for the slot's token; beside other tokens it is a bad id
    code, _, _, got, layout = _pack(**dict(base, tokens=[5, 6, DEVICE_TOKEN]))
    assert code == 0 and got[layout.offsets()["token_ids"][0] + 2] == -(1 + 1)
    code, bad, err, *_ = _pack(**dict(base, tokens=[DEVICE_TOKEN, 6, 7]))
    assert (code, bad) == (2, 0)
