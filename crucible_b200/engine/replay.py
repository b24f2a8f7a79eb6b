"""Trace replay: feeds given token ids through the engine step by step and
writes the logits.  It samples nothing and has no forward pass, cache or loader
of its own: it drives `Engine.step`, the same function generation uses.

Input: one JSON object a line on standard input,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` receives the logits
at the wanted places (order of the entries, then of `want`) as little-endian
float32 [wanted, vocab].  After every step a line `done <step>` is printed and
flushed.  Requests named in `end` give back what they hold after the step.

The reference's nearest tools are `scripts/reference_logits.py:37-63` (tokens ->
last-position logits) and `llm-engine gpu-logits` (`engine/src/main.rs:1006`).
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np

from ..ops import tensor_core
from .engine import Engine, EngineOptions, StepEntry


def make_engine(model_dir: str, dtype: str, max_tokens: int, page_tokens: int = 16,
                max_requests: int = 4) -> Engine:
    """An engine whose cache pool holds `max_tokens` tokens, each request's
    count rounded up to a multiple of 64 by the caller's contract (64 is a
    multiple of the page size, so the pool is max_tokens / page_tokens pages)."""
    if max_tokens <= 0:
        raise ValueError("--max-tokens must be positive")
    unit = 64 if 64 % page_tokens == 0 else page_tokens
    tokens = -(-max_tokens // unit) * unit
    n_pages = -(-tokens // page_tokens)
    return Engine(model_dir, EngineOptions(dtype=dtype, page_tokens=page_tokens,
                                           n_pages=n_pages, max_requests=max_requests))


def run(engine: Engine, lines: IO[str], out_dir: str, done: Optional[IO[str]] = None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    done = done if done is not None else sys.stdout
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                host = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                # the copy waited for the step; a kernel that gave up a wait says so now,
                # before anything of this step is written
                tensor_core.check_status(engine.device)
                host.tofile(os.path.join(out_dir, f"{step}.f32"))
        for req in rec.get("end", []):
            engine.finish(req)
        done.write(f"done {step}\n")
        done.flush()
        n += 1
    tensor_core.check_status(engine.device)      # steps that wanted nothing were not waited for
    return n


def main(argv=None) -> int:
    import argparse
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--page-tokens", type=int, default=16, help="tokens per cache page")
    args = p.parse_args(argv)
    engine = make_engine(args.model, args.dtype, args.max_tokens, args.page_tokens)
    run(engine, sys.stdin, args.out)
    return 0
