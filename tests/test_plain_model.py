"""The plain implementation against the reference's own PyTorch model (golden
files made by tests/golden/make_golden.py), and the plain sampler's rules."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_model as pm
from crucible_b200.sampling import SamplingParams, Xorshift64Star

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["golden_a", "golden_b"])
def test_plain_forward_matches_the_reference_model(name):
    folder = os.path.join(GOLDEN, name)
    cfg, w = pm.read_folder(folder)
    tokens = json.load(open(os.path.join(folder, "tokens.json")))
    want = np.load(os.path.join(folder, "logits.npy")).astype(np.float64)
    got = pm.plain_forward(cfg, w, tokens).numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 5e-6 * np.abs(want).max()


def test_plain_forward_is_causal():
    cfg, w = pm.read_folder(os.path.join(GOLDEN, "golden_a"))
    tokens = json.load(open(os.path.join(GOLDEN, "golden_a", "tokens.json")))
    base = pm.plain_forward(cfg, w, tokens)
    changed = list(tokens)
    changed[10] = (changed[10] + 1) % cfg["vocab"]
    other = pm.plain_forward(cfg, w, changed)
    assert torch.equal(base[:10], other[:10]) and not torch.equal(base[10:], other[10:])


def test_parts_one_by_one():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = pm.plain_rmsnorm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]], dtype=torch.float64))
    cos, sin = pm.plain_rope_tables(4, 3, 100.0)
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=torch.float64).repeat(3, 1, 1)
    r = pm.plain_rope(v, cos, sin)
    assert torch.allclose(r[0], v[0])                                        # position 0: identity
    a1 = 1.0                                                                 # pos 1, freq 100^0
    assert r[1, 0, 0] == pytest.approx(1 * math.cos(a1) - 3 * math.sin(a1))  # pairs (0,2) and (1,3)
    assert r[1, 0, 2] == pytest.approx(1 * math.sin(a1) + 3 * math.cos(a1))
    assert r[1, 0, 1] == pytest.approx(2 * math.cos(0.1) - 4 * math.sin(0.1))
    q = torch.zeros(2, 2, 2, dtype=torch.float64)
    k = torch.zeros(2, 1, 2, dtype=torch.float64)
    vv = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=torch.float64)
    o = pm.plain_attention(q, k, vv)
    assert torch.allclose(o[0], torch.tensor([[1.0, 0.0]] * 2, dtype=torch.float64))    # sees itself only
    assert torch.allclose(o[1], torch.tensor([[0.5, 0.5]] * 2, dtype=torch.float64))    # both heads, one KV head
    o_w = pm.plain_attention(q, k, vv, window=1)
    assert torch.allclose(o_w[1], torch.tensor([[0.0, 1.0]] * 2, dtype=torch.float64))


def test_generators_agree_and_match_the_formula():
    a, b = pm.PlainRng(1234), Xorshift64Star(1234)
    xs = [a.next_f32() for _ in range(100)]
    assert xs == [b.next_f32() for _ in range(100)]
    assert all(0.0 <= x < 1.0 for x in xs) and len(set(xs)) > 90
    s = 1234 | 1
    s ^= s >> 12
    s ^= (s << 25) & (2 ** 64 - 1)
    s ^= s >> 27
    assert xs[0] == ((s * 0x2545F4914F6CDD1D % 2 ** 64) >> 40) / 2 ** 24
    assert pm.PlainRng(0).s == 1                                   # seed | 1: zero is a fixed point


def test_sampler_rules():
    nan = float("nan")
    assert pm.plain_argmax([1.0, 3.0, 3.0]) == 1                   # lowest index among maxima
    assert pm.plain_argmax([1.0, nan, 0.5]) == 0                   # NaN never displaces
    assert [i for i, _ in pm.plain_top_k([0.5, 2.0, nan, 2.0, 1.0], 3)] == [1, 3, 4]
    assert len(pm.plain_top_k([1.0, 2.0], 0)) == 1                 # top_k clamps to [1, V]
    assert len(pm.plain_top_k([1.0, 2.0], 99)) == 2
    rng = pm.PlainRng(7)
    state = rng.s
    assert pm.plain_sample([0.1, 0.9, 0.3], 0.0, 40, rng) == 1 and rng.s == state   # greedy draws nothing
    assert pm.plain_sample([0.1, 0.9, 0.3], 0.7, 1, rng) == 1 and rng.s != state    # k = 1: the best
    counts = [0, 0, 0]
    rng = pm.PlainRng(3)
    for _ in range(3000):
        counts[pm.plain_sample([0.0, math.log(2.0), -50.0], 1.0, 3, rng)] += 1
    assert counts[2] == 0 and 1.7 < counts[1] / counts[0] < 2.3
    assert pm.plain_sample([nan, nan], 0.8, 2, pm.PlainRng(1)) == 0                # nothing finite: best


def test_sampling_params():
    p = SamplingParams()
    assert (p.max_tokens, p.temperature, p.top_k, p.seed, p.is_greedy) == (64, 0.0, 40, 1234, True)
    assert SamplingParams(top_k=0).effective_top_k(100) == 1
    assert SamplingParams(top_k=500).effective_top_k(100) == 100
    with pytest.raises(ValueError):
        SamplingParams(temperature=101.0).validate(100)
    with pytest.raises(ValueError):
        SamplingParams(max_tokens=0).validate(100)
    with pytest.raises(ValueError, match="top_k"):
        SamplingParams(temperature=0.8, top_k=5000).validate(50000, max_device_top_k=1024)
    SamplingParams(temperature=0.0, top_k=5000).validate(50000, max_device_top_k=1024)
