"""The command line, in the reference's manner (`engine/src/main.rs:24-498`).

    llm-engine generate MODEL --prompt-ids 1,2,3 [--max-tokens 40] [--temperature 0.8]
                              [--top-k 40] [--seed 1234] [--graph] [--dtype bfloat16]
    llm-engine inspect MODEL
    llm-engine logits MODEL --tokens 1,2,3 [--top 10]
    llm-engine random-weights --shape 120m --seed 0 OUT

`generate` keeps the reference's option names, defaults and meanings
(`main.rs:476-497`: --max-tokens 40, --temperature 0.8, --top-k 40, --seed 1234,
--gpu, --graph).  The reference's tokenizer is outside this engine's contract:
prompts are token ids (`--prompt-ids`, or `--prompt-len N` for seeded random
ids).  `--gpu` is accepted and means nothing: there is no CPU path.  `inspect`
follows `main.rs:943-1002`, `logits` follows `main.rs:905-941` and
`scripts/reference_logits.py:49-63` (sum, min, max, ordered top-N of the
last position).
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time


def _ids(text: str):
    try:
        return [int(x) for x in text.replace(" ", "").split(",") if x != ""]
    except ValueError:
        raise SystemExit(f"token ids must be integers separated by commas, got {text!r}")


def _add_engine_options(p):
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max-batch", type=int, default=16, help="requests resident at once")
    p.add_argument("--kv-pages", type=int, default=None,
                   help="KV pages; default: enough for max-batch full-context sequences")
    p.add_argument("--page-tokens", type=int, default=16, help="tokens per KV page")
    p.add_argument("--prefill-chunk-tokens", type=int, default=None,
                   help="cap on one request's prompt tokens per scheduler step")
    p.add_argument("--prefill-token-budget", type=int, default=1024,
                   help="tokens per scheduler step")
    p.add_argument("--max-prefill-requests", type=int, default=None)


def cmd_generate(args) -> int:
    from ..sampling.params import SamplingParams
    from .llm import LLM
    llm = LLM(args.model, dtype=args.dtype, max_batch=args.max_batch, kv_pages=args.kv_pages,
              page_tokens=args.page_tokens, prefill_token_budget=args.prefill_token_budget,
              prefill_chunk_tokens=args.prefill_chunk_tokens,
              max_prefill_requests=args.max_prefill_requests, graph=args.graph,
              profile=args.profile)
    vocab = llm.config.vocab_size
    if args.prompt_ids is not None:
        prompts = [_ids(p) for p in args.prompt_ids]
    else:
        rng = random.Random(args.seed_ids)
        prompts = [[rng.randrange(vocab) for _ in range(args.prompt_len)]
                   for _ in range(args.n_prompts)]
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature,
                            top_k=args.top_k, seed=args.seed, eos_token_id=args.eos_token_id)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params)
    dt = time.perf_counter() - t0
    for i, (prompt, out) in enumerate(zip(prompts, outs)):
        print(json.dumps({"request": i, "prompt_tokens": len(prompt), "tokens": out}))
    prefill = sum(s.prefill_tokens for s in llm.last_steps)
    decoded = sum(s.decoded for s in llm.last_steps)
    t_pre = sum(s.wall_s for s in llm.last_steps if s.prefill_tokens)
    t_dec = sum(s.wall_s for s in llm.last_steps if not s.prefill_tokens)
    print(f"prefill: {prefill} tokens in {t_pre * 1e3:.1f} ms"
          + (f" ({prefill / t_pre:.0f} tok/s)" if t_pre > 0 else ""), file=sys.stderr)
    print(f"decode: {decoded} tokens in {t_dec * 1e3:.1f} ms"
          + (f" ({decoded / t_dec:.0f} tok/s)" if t_dec > 0 else ""), file=sys.stderr)
    if args.verbose:
        for s in llm.last_steps:
            print(json.dumps(s.__dict__), file=sys.stderr)
    print(f"total {dt * 1e3:.1f} ms, {len(llm.last_steps)} steps", file=sys.stderr)
    if llm.engine.profiler is not None:
        print(llm.engine.profiler.text(), file=sys.stderr)
    return 0


def cmd_inspect(args) -> int:
    from ..config.registry import load_config
    from ..models.decoder import DecoderModel
    from ..weights.safetensors_io import SafetensorsFile
    import os
    cfg = load_config(args.model)
    model = DecoderModel(cfg)
    m = cfg.layers[0].mixer
    print(f"architecture   {cfg.architecture}")
    print(f"layers         {cfg.n_layers} (run order of {len(cfg.run_order)})")
    print(f"width          {cfg.hidden_size}")
    print(f"vocabulary     {cfg.vocab_size} ({'tied' if cfg.tie_word_embeddings else 'untied'} head)")
    print(f"context        {cfg.max_context}")
    print(f"layer 0 mixer  {m.kind}: {m.n_heads} heads, {m.n_kv_heads} kv heads, head size "
          f"{m.head_dim}, window {m.window}")
    print(f"layer 0 ffn    {cfg.layers[0].feed_forward.kind}: {cfg.layers[0].feed_forward.intermediate}")
    print(f"norm           {cfg.final_norm.kind} eps {cfg.final_norm.eps}")
    print(f"cache groups   {len(model.cache_groups)}; state bytes per request {model.state_bytes}")
    f = SafetensorsFile(os.path.join(args.model, "model.safetensors"))
    total = 0
    for name in sorted(f.names()):
        e = f.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        total += n
        if args.tensors:
            print(f"  {name:60s} {e.dtype:5s} {list(e.shape)}")
    print(f"tensors        {len(f.names())}, {total / 1e6:.2f} M values")
    f.close()
    return 0


def cmd_logits(args) -> int:
    import torch
    from .engine import Engine, EngineOptions, StepEntry
    tokens = _ids(args.tokens)
    engine = Engine(args.model, EngineOptions(dtype=args.dtype, max_requests=1,
                                              n_pages=-(-len(tokens) // 16) + 1, graph=False))
    logits = engine.step([StepEntry("r", tokens, [len(tokens) - 1])])[0].double().cpu()
    print(f"tokens {tokens}")
    print(f"logits: sum {logits.sum().item():.4f}, min {logits.min().item():.6f}, "
          f"max {logits.max().item():.6f}")
    print()
    print(f"top {args.top}:")
    values, indices = torch.topk(logits, min(args.top, logits.numel()))
    for i, v in zip(indices.tolist(), values.tolist()):
        print(f"  {i:6} {v:10.6f}")
    return 0


def cmd_random_weights(args) -> int:
    from ..config.presets import shape
    from ..weights.random_init import write_random_model
    if args.config:
        with open(args.config) as f:
            raw = json.load(f)
    else:
        raw = shape(args.shape)
    out = write_random_model(raw, args.out, args.seed, std=args.std, store_dtype=args.store_dtype)
    print(f"wrote {out}")
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="llm-engine")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids from prompts of token ids")
    g.add_argument("model")
    g.add_argument("--prompt-ids", action="append", default=None,
                   help="comma-separated token ids; repeat for several prompts")
    g.add_argument("--prompt-len", type=int, default=16)
    g.add_argument("--n-prompts", type=int, default=1)
    g.add_argument("--seed-ids", type=int, default=1)
    g.add_argument("--max-tokens", type=int, default=40)
    g.add_argument("--temperature", type=float, default=0.8)
    g.add_argument("--top-k", type=int, default=40)
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--eos-token-id", type=int, default=None)
    g.add_argument("--gpu", action="store_true", help="accepted; this engine always runs on the GPU")
    g.add_argument("--graph", action="store_true", default=True,
                   help="replay decode steps from captured CUDA graphs (default)")
    g.add_argument("--no-graph", dest="graph", action="store_false")
    g.add_argument("--verbose", action="store_true", help="print every scheduler step")
    g.add_argument("--profile", action="store_true",
                   help="time every part of the model with CUDA events (steps run eagerly) and "
                        "print the stage table")
    _add_engine_options(g)
    g.set_defaults(func=cmd_generate)

    i = sub.add_parser("inspect", help="print the configuration and tensor inventory")
    i.add_argument("model")
    i.add_argument("--tensors", action="store_true")
    i.set_defaults(func=cmd_inspect)

    l = sub.add_parser("logits", help="last-position logits of a token sequence")
    l.add_argument("model")
    l.add_argument("--tokens", default="464,2159,318,1719")
    l.add_argument("--top", type=int, default=10)
    l.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    l.set_defaults(func=cmd_logits)

    r = sub.add_parser("random-weights", help="write a model folder with random weights")
    r.add_argument("out")
    r.add_argument("--shape", default="120m")
    r.add_argument("--config", default=None, help="a config.json to use instead of a named shape")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(func=cmd_random_weights)

    args = p.parse_args(argv)
    return args.func(args)
