"""Shared by the tests: tiny model folders, traces, and the comparison rule."""
from __future__ import annotations

import io
import json
import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

# Tiny configurations (the first two differ in every size and option: layers, width,
# head counts and group size, head size, feed-forward width, vocabulary, rotary
# base, norm epsilon, tied or untied head, context, and (below) the page size).
TINY = {
    "tiny-a": dict(config={
        "architectures": ["CrucibleGPT"], "vocab_size": 256, "n_layer": 2, "n_head": 4,
        "n_kv_head": 2, "n_embd": 64, "head_dim": 16, "intermediate_size": 176,
        "block_size": 512, "attention": "gqa", "pos_encoding": "rope", "activation": "swiglu",
        "norm": "rmsnorm", "norm_placement": "pre", "rope_theta": 10000.0,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True}, seed=0, page_tokens=16),
    "tiny-b": dict(config={
        "architectures": ["LlamaForCausalLM"], "vocab_size": 509, "num_hidden_layers": 3,
        "num_attention_heads": 3, "num_key_value_heads": 1, "hidden_size": 96, "head_dim": 32,
        "intermediate_size": 320, "max_position_embeddings": 448, "hidden_act": "silu",
        "rope_theta": 500000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False},
        seed=2, page_tokens=32),
    # head size 64: the bfloat16 engine then runs its tcgen05 attention kernels and the
    # q/k/v product with the rotation in its epilogue; the q width differs from the model's
    "tiny-c": dict(config={
        "architectures": ["LlamaForCausalLM"], "vocab_size": 300, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": 128, "head_dim": 64,
        "intermediate_size": 208, "max_position_embeddings": 512, "hidden_act": "silu",
        "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True},
        seed=5, page_tokens=16),
}

# Larger than the reference's 0.02 so that attention is not nearly uniform and
# a wrong key, page or position moves the logits well above rounding.
TEST_STD = 0.08

# The comparison rule, fixed before any kernel was written: the largest
# absolute difference over a request's logits, relative to the largest
# reference logit of that request.
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}


def make_folder(tmp_path, name: str) -> str:
    from crucible_b200.weights import write_random_model
    out = os.path.join(str(tmp_path), name)
    write_random_model(TINY[name]["config"], out, TINY[name]["seed"], std=TEST_STD)
    return out


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def plain_logits(model_dir: str, tokens: Sequence[int]) -> np.ndarray:
    import plain_model as pm
    cfg, w = pm.read_folder(model_dir)
    return pm.plain_forward(cfg, w, tokens).to(torch.float64).numpy()


def relative_error(got: np.ndarray, ref: np.ndarray) -> float:
    scale = max(float(np.abs(ref).max()), 1e-6)
    return float(np.abs(got.astype(np.float64) - ref).max()) / scale


class Trace:
    """Builds trace steps and remembers which (request, position) each wanted row is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.wanted: List[List[Tuple[str, int]]] = []
        self._fed: Dict[str, int] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]],
             end: Sequence[str] = ()) -> None:
        recs, wanted = [], []
        for rid, tokens, want in entries:
            start = self._fed.get(rid, 0)
            recs.append({"id": rid, "tokens": list(tokens), "want": list(want)})
            wanted.extend((rid, start + w) for w in want)
            self._fed[rid] = start + len(tokens)
        for rid in end:
            self._fed.pop(rid, None)
        self.steps.append({"step": len(self.steps), "entries": recs, "end": list(end)})
        self.wanted.append(wanted)

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def collect(trace: Trace, out_dir: str, vocab: int) -> Dict[Tuple[str, int], np.ndarray]:
    """(request, position) -> logits row, from the files a replay wrote."""
    got = {}
    for i, wanted in enumerate(trace.wanted):
        path = os.path.join(out_dir, f"{i}.f32")
        if not wanted:
            assert not os.path.exists(path), f"step {i} wanted nothing but wrote a file"
            continue
        data = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
        for row, key in zip(data, wanted):
            got[key] = row
    return got


def replay_in_process(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int,
                      page_tokens: int):
    from crucible_b200.engine import replay
    engine = replay.make_engine(model_dir, dtype, max_tokens, page_tokens)
    done = io.StringIO()
    replay.run(engine, io.StringIO(trace.text()), out_dir, done)
    assert done.getvalue().split() == [x for i in range(len(trace.steps)) for x in ("done", str(i))]
    engine.cache.check_invariants()
    return engine
