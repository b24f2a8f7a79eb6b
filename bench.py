#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second (a "step" is
one decode step) and prefill tokens per second, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference|cpu]

Default run: the layer sizes of the 120M shape (12 layers, width 768, 12 query
and 4 KV heads of size 64, SwiGLU 2048, vocabulary 50,304, tied head) with
random bfloat16 weights, batch 8, 2,048-token contexts.  It prints ONE JSON
line.  `value` is decoded tokens per second through the engine's step function
with the chosen ids fed back on the device (K timed steps bracketed by CUDA
events); `e2e` is the same through the Python entry point `LLM.generate`, host
token ids in and out; `prefill` is a 2,048-token prompt in one step (eight such
steps timed as a run, `ms` is one step's share);
`points` are decode at batch 1 and 64; `roofline` relates the decode step to
the measured HBM bandwidth.  Token ids are uniform random with a fixed seed and
the weights are N(0, 0.02) from seed 0: the data is synthetic.

For --gpus N > 1 it prints one line that says so and exits with 2: this engine
runs on one GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REFERENCE_DIR = os.path.join(ROOT, "baseline", "_ref")
REFERENCE_NOTE = ("the reference's engine is Rust with NVRTC kernels for sm_120 (no cargo in this "
                  "image, not installable by pip); this arm runs the reference's own PyTorch model, "
                  "an unmodified copy of its model.py, through its GPT.forward / GPT.generate")


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while work runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self._stop = threading.Event()
        self._thread = None
        self._proc = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            if self._stop.is_set():
                break
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.time(), parts))

    def stop(self):
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

    def summary(self, windows):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, parts in self.samples:
            if windows and not any(a <= t <= b for a, b in windows):
                continue
            try:
                sm.append(int(float(parts[0])))
                mx = max(mx, int(float(parts[1])))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            for t, parts in self.samples:
                try:
                    sm.append(int(float(parts[0])))
                    mx = max(mx, int(float(parts[1])))
                except ValueError:
                    pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg):
    """Matrix elements and cache bytes of the model as its run order says: every entry of
    the run order counts with its own layer's sizes (layers may differ, run twice, or read
    another layer's cache, in which case they keep none of their own)."""
    d, V = cfg.hidden_size, cfg.vocab_size
    weights = attn_width = kv_token_bytes = 0
    for entry in cfg.run_order:
        layer = cfg.layers[entry.layer]
        m, f = layer.mixer, layer.feed_forward
        weights += (d * m.n_heads * m.head_dim + 2 * d * m.n_kv_heads * m.head_dim
                    + m.n_heads * m.head_dim * d + 3 * d * f.intermediate)
        attn_width += m.n_heads * m.head_dim
        if entry.cache_of is None:
            kv_token_bytes += 2 * m.n_kv_heads * m.head_dim * 2
    return dict(layer_weights=weights, head=V * d, layers=len(cfg.run_order),
                kv_token_bytes=kv_token_bytes, attn_width=attn_width)


def prefill_flops(nums, t):
    gemm = 2 * t * nums["layer_weights"] + 2 * nums["head"]
    attn = 2 * 2 * nums["attn_width"] * t * (t + 1) // 2
    return gemm + attn


SHAPE_LABEL = {"120m": "120M", "llama-1b": "Llama-3.2-1B", "llama-8b": "Llama-3-8B"}


def run_ours(args):
    import torch
    from crucible_b200 import LLM, SamplingParams, ops
    from crucible_b200.config import parse_config, shape
    from crucible_b200.engine import DEVICE_TOKEN, StepEntry
    from crucible_b200.ops import tensor_core
    from crucible_b200.weights import write_random_model

    peaks = read_peaks()
    raw = shape(args.shape)
    layer_key = "n_layer" if "n_layer" in raw else "num_hidden_layers"
    full_layers = raw[layer_key]
    if args.layers:
        raw[layer_key] = args.layers
    cfg = parse_config(raw)
    nums = model_numbers(cfg)
    ctx_len, batch, new_tokens = args.context, args.batch, args.steps
    rng = random.Random(1)
    vocab = cfg.vocab_size

    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(raw, os.path.join(tmp, "model"), seed=0)
        max_batch = 64
        page = 16
        need_tokens = max(ctx_len + args.steps + args.warmup + 64, cfg.max_context)
        kv_pages = max_batch * (-(-need_tokens // page)) + 64
        llm = LLM(folder, dtype="bfloat16", max_batch=max_batch, kv_pages=kv_pages,
                  page_tokens=page, prefill_token_budget=2048)
    engine = llm.engine
    dev = engine.device
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def prompt(n):
        return [rng.randrange(vocab) for _ in range(n)]

    # ---- prefill: one 2,048-token prompt, one step --------------------------------
    # Timed like the decode steps: a run of steps between two events, each a fresh request
    # that is finished before the next, so that the host's preparation of a step runs under
    # the device's work on the step before (one step alone would count the host's part too).
    t_prefill = 2048
    n_prefill = 8
    prompts = [prompt(t_prefill) for _ in range(args.warmup + n_prefill)]
    for tokens in prompts[:args.warmup]:
        engine.step([StepEntry("p", tokens, [t_prefill - 1])])
        engine.finish("p")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    w0 = time.time()
    e0.record()
    for tokens in prompts[args.warmup:]:
        engine.step([StepEntry("p", tokens, [t_prefill - 1])])
        engine.finish("p")
    e1.record()
    torch.cuda.synchronize()
    windows.append((w0, time.time()))
    prefill_ms = e0.elapsed_time(e1) / n_prefill
    prefill_tflops = prefill_flops(nums, t_prefill) / (prefill_ms / 1e3) / 1e12
    prefill = {"value": round(t_prefill / (prefill_ms / 1e3), 1), "tokens": t_prefill,
               "ms": round(prefill_ms, 4), "steps": n_prefill,
               "frac": round(prefill_tflops / peaks["bf16_tflops"], 4),
               "frac_of_sustained": round(prefill_tflops / peaks["bf16_tflops_sustained"], 4),
               "tflops": round(prefill_tflops, 1)}

    # ---- decode through the step function -------------------------------------------
    def decode_run(b, steps, warmup, ctx_len=ctx_len):
        ids = [f"d{i}" for i in range(b)]
        for rid in ids:
            engine.step([StepEntry(rid, prompt(ctx_len - 1), [])])
        # The decode step as generation runs it: the step chooses its tokens itself
        # (`Engine.step_choosing`: greedy, the argmax captured with the step), a chosen token
        # stays on the device as the request's next one (an entry of DEVICE_TOKEN), and its id
        # travels to the host beside the next step and is read one step late.
        in_flight = [engine.step_choosing([StepEntry(rid, [rng.randrange(vocab)], [0]) for rid in ids])[1]]
        entries = [StepEntry(rid, [DEVICE_TOKEN], [0]) for rid in ids]

        def one():
            in_flight.append(engine.step_choosing(entries)[1])
            in_flight.pop(0).get()
        for _ in range(warmup - 1):
            one()
        torch.cuda.synchronize()
        launches0 = ops.LAUNCHES[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        ms = e0.elapsed_time(e1)
        launches = ops.LAUNCHES[0] - launches0
        tensor_core.check_status(dev)
        first_ctx = ctx_len + warmup
        mean_ctx = first_ctx + (steps - 1) / 2.0
        for rid in ids:
            engine.finish(rid)
        return dict(tok_s=b * steps / (ms / 1e3), ms_per_step=ms / steps, launches=launches,
                    mean_ctx=mean_ctx)

    weight_bytes = (nums["layer_weights"] + nums["head"]) * 2

    def hbm_gbs(r, b):
        """Bytes a decode step has to read (every weight once, the live requests' cache
        at the run's mean context) over its time."""
        return (weight_bytes + b * r["mean_ctx"] * nums["kv_token_bytes"]) / (r["ms_per_step"] / 1e3) / 1e9

    main = decode_run(batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        r = decode_run(b, args.steps, args.warmup)
        points[f"decode_b{b}"] = round(r["tok_s"], 1)
        points[f"decode_b{b}_ms"] = round(r["ms_per_step"], 4)
        points[f"decode_b{b}_frac"] = round(hbm_gbs(r, b) / peaks["hbm_gbs"], 4)

    # further batches and context lengths of the same model (the hand-over between the
    # few-row kernels and the tiles at 16 / 32 rows; short and long contexts)
    steps_more = min(args.steps, 64)
    for b, c in ((16, ctx_len), (32, ctx_len), (8, 512), (64, 512), (8, cfg.max_context - 320),
                 (64, cfg.max_context - 320)):
        if c + steps_more + args.warmup + 1 > cfg.max_context or c <= 0:
            continue
        r = decode_run(b, steps_more, args.warmup, ctx_len=c)
        key = f"decode_b{b}" + ("" if c == ctx_len else f"_ctx{c}")
        points[key + "_ms"] = round(r["ms_per_step"], 4)
        points[key + "_frac"] = round(hbm_gbs(r, b) / peaks["hbm_gbs"], 4)

    # ---- a mixed step: 63 requests decoding beside one 512-token portion ----------------
    # (the decoded tokens go through the split attention kernel, the portion through the
    # tile kernel, in one step); beside it, for comparison, the 512-token portion alone.
    def mixed_run(n_decoding, portion, steps, warmup):
        ids = [f"m{i}" for i in range(n_decoding)]
        for rid in ids:
            engine.step([StepEntry(rid, prompt(ctx_len - 1), [])])
        decoding = [StepEntry(rid, [rng.randrange(vocab)], [0]) for rid in ids]
        portions = [prompt(portion) for _ in range(warmup + steps)]

        def one(tokens):
            engine.step(decoding + [StepEntry("fresh", tokens, [portion - 1])])
            engine.finish("fresh")
        for tokens in portions[:warmup]:
            one(tokens)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        w0 = time.time()
        e0.record()
        for tokens in portions[warmup:]:
            one(tokens)
        e1.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        for rid in ids:
            engine.finish(rid)
        return e0.elapsed_time(e1) / steps

    points["mixed_63_decoding_plus_512_ms"] = round(mixed_run(63, 512, 16, args.warmup), 4)
    points["portion_512_alone_ms"] = round(mixed_run(0, 512, 16, args.warmup), 4)

    achieved = hbm_gbs(main, batch)
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                "peaks": peaks["source"]}

    # ---- end to end through the Python entry point -----------------------------------
    def through_generate(n_req, pure_steps):
        """Tokens/s over the iterations in which all `n_req` requests decode and no prompt is
        in work.  Prompts enter one per step (the token budget), so the first request has
        decoded n_req - 1 tokens beside the others' prompts before the last one joins:
        that many tokens more are asked for."""
        # untimed: the same batch for a few steps, so that every shape of step the timed run
        # replays has been captured (a capture costs the host 4 ms, once per shape and
        # metadata buffer)
        llm.generate([prompt(ctx_len) for _ in range(n_req)], SamplingParams(max_tokens=n_req + max(3, args.warmup)))
        prompts = [prompt(ctx_len) for _ in range(n_req)]
        w0 = time.time()
        outs = llm.generate(prompts, SamplingParams(max_tokens=pure_steps + n_req))
        windows.append((w0, time.time()))
        assert all(len(o) == pure_steps + n_req for o in outs)
        chosen = [s for s in llm.last_steps if s.prefill_tokens == 0 and s.decoded == n_req]
        wall = sum(s.wall_s for s in chosen)
        return (len(chosen) * n_req / wall if wall > 0 else 0.0), chosen

    llm.generate([prompt(ctx_len)], SamplingParams(max_tokens=2))          # warm the path
    e2e_tok_s, decode_steps = through_generate(batch, args.steps)
    if batch != 64:
        points["e2e_b64"] = round(through_generate(64, 16)[0], 1)
    h2d = 0
    if decode_steps:
        from crucible_b200.engine.context import StepLayout
        # the step's metadata block (greedy requests upload nothing else: the sampler's row of
        # state slots goes up only when it changes); back come the chosen ids and the status
        # word behind them
        h2d = StepLayout(batch, batch, batch, engine.table_strides).offsets()["_total"][1] * 4
    e2e = {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4 * (batch + 1), "steps": len(decode_steps)}

    clocks.stop()
    line = {
        "metric": f"decode tok/s at batch {batch} ({SHAPE_LABEL[args.shape]} shape, bf16, "
                  f"{ctx_len:,}-token contexts)",
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"crucible-{args.shape}-shape", "layers": nums["layers"],
                   "layers_of_shape": full_layers, "hidden": cfg.hidden_size,
                   "q_heads": cfg.layers[0].mixer.n_heads,
                   "kv_heads": cfg.layers[0].mixer.n_kv_heads,
                   "head_dim": cfg.layers[0].mixer.head_dim,
                   "intermediate": cfg.layers[0].feed_forward.intermediate,
                   "vocab": cfg.vocab_size, "tied_head": cfg.tie_word_embeddings,
                   "global_batch": batch, "seq_len": ctx_len, "new_tokens": args.steps,
                   "kv_page_tokens": 16, "parallelism": "single-gpu",
                   "l2": "inputs_exceed_l2", "weights": "random N(0,0.02) seed 0"},
        "e2e": e2e, "gpu_launches": main["launches"], "prefill": prefill,
        "roofline": roofline, "points": points, "clocks": clocks.summary(windows),
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    """The reference arm: the reference's own PyTorch model (`model.py`, copied unmodified
    to baseline/_ref/) at the same shape, batch and context, through its stock code path:
    `GPT.generate` (`model.py:371-383`, which runs the whole sequence again for every new
    token: it keeps no cache) for decoding and `GPT.forward` (`model.py:343-365`) for the
    prefill.  Nothing of crucible_b200 is imported here and none of its libraries is
    loaded."""
    path = os.path.join(REFERENCE_DIR, "model.py")
    if not os.path.exists(path):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref/model.py is absent (copy the reference's model.py "
                          "there); " + REFERENCE_NOTE}))
        return 0
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location("crucible_reference_model", path)
    ref = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = ref
    spec.loader.exec_module(ref)
    if args.shape != "120m":
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the reference arm runs the 120M shape only, not {args.shape}"}))
        return 0
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    layers = args.layers or 12
    cfg = ref.GPTConfig(vocab_size=50304, n_layer=layers, n_head=12, n_kv_head=4, n_embd=768,
                        block_size=4096, attention="gqa")
    model = ref.GPT(cfg).to(dev).to(torch.bfloat16).eval()
    batch, ctx_len, steps, warmup = args.batch, args.context, args.steps, max(3, args.warmup)
    gen = torch.Generator().manual_seed(1)
    peaks = read_peaks()
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def ids(b, n):
        return torch.randint(0, cfg.vocab_size, (b, n), generator=gen, dtype=torch.long)

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        w0 = time.time()
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        return e0.elapsed_time(e1), out

    with torch.no_grad():
        # prefill: one 2,048-token forward (logits at the last position only)
        t_prefill, n_prefill = 2048, 8
        prompts = [ids(1, t_prefill).to(dev) for _ in range(warmup + n_prefill)]
        for x in prompts[:warmup]:
            model(x)
        ms, _ = timed(lambda: [model(x) for x in prompts[warmup:]])
        prefill_ms = ms / n_prefill
        d, inter = 768, 64 * ((int(2 * (4 * 768) / 3) + 63) // 64)
        per_layer = d * 768 + 2 * d * 256 + 768 * d + 3 * d * inter
        flops = (2 * t_prefill * layers * per_layer + 2 * 50304 * d
                 + layers * 2 * 2 * 768 * t_prefill * (t_prefill + 1) // 2)
        prefill = {"value": round(t_prefill / (prefill_ms / 1e3), 1), "tokens": t_prefill,
                   "ms": round(prefill_ms, 4), "steps": n_prefill,
                   "frac": round(flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}

        def decode(b, k):
            start = ids(b, ctx_len).to(dev)
            model.generate(start, warmup, temperature=1.0, top_k=1)
            ms, _ = timed(lambda: model.generate(start, k, temperature=1.0, top_k=1))
            return b * k / (ms / 1e3), ms / k

        tok_s, ms_per_step = decode(batch, steps)
        points = {}
        for b in (1, 64):
            k = min(steps, 16)              # a step of the reference costs b x 2,048 tokens
            r = decode(b, k)
            points[f"decode_b{b}"] = round(r[0], 1)
            points[f"decode_b{b}_ms"] = round(r[1], 4)
        # end to end: host ids in (pinned), host ids out, around the same generate call
        host = ids(batch, ctx_len).pin_memory()
        t0 = time.time()
        out = model.generate(host.to(dev, non_blocking=True), steps, temperature=1.0, top_k=1).cpu()
        wall = time.time() - t0
        windows.append((t0, time.time()))
        assert out.shape == (batch, ctx_len + steps)
    clocks.stop()
    weight_bytes = (layers * per_layer + 50304 * d) * 2
    kv_token_bytes = 2 * 256 * layers * 2
    achieved = (weight_bytes + batch * (ctx_len + warmup + (steps - 1) / 2.0) * kv_token_bytes) \
        / (ms_per_step / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {batch} (120M shape, bf16, {ctx_len:,}-token contexts)",
        "value": round(tok_s, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference", "note": REFERENCE_NOTE + "; weights cast to bfloat16, greedy "
                                     "(top_k=1), no KV cache in its generate",
        "config": {"model": "crucible-120m-shape", "layers": layers, "layers_of_shape": 12,
                   "hidden": 768, "q_heads": 12, "kv_heads": 4, "head_dim": 64,
                   "intermediate": inter, "vocab": 50304, "tied_head": True,
                   "global_batch": batch, "seq_len": ctx_len, "new_tokens": steps,
                   "kv_page_tokens": 0, "parallelism": "single-gpu", "l2": "inputs_exceed_l2",
                   "weights": "random N(0,0.02) seed 0 (its own init)"},
        "e2e": {"value": round(batch * steps / wall, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": batch * ctx_len * 8 // steps,
                "d2h_bytes_per_step": batch * (ctx_len + steps) * 8 // steps, "steps": steps},
        "gpu_launches": 0, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                     "peaks": peaks["source"]},
        "points": points, "clocks": clocks.summary(windows),
    }
    print(json.dumps(line))
    return 0


def run_cpu_baseline(args):
    """A timed CPU baseline: a plain float32 forward of whole sequences (no cache, no
    batching; embedding, RMSNorm, half-split RoPE, grouped-query attention, SwiGLU, tied
    or untied head, written here from the model's formulas with torch's CPU operators) on
    the two tiny shapes and on one layer of the 120M shape.  The reference's own scalar
    CPU engine decodes 9.66 tokens/s on its 120M model (`README.md:486-490`); this is the
    number to hold the GPU figures against on the machine at hand."""
    import math
    import torch
    from crucible_b200.config import parse_config, shape
    torch.manual_seed(0)

    def forward(cfg, weights, tokens):
        layer0 = cfg.layers[0]
        m, f = layer0.mixer, layer0.feed_forward
        hq, hkv, hd, t = m.n_heads, m.n_kv_heads, m.head_dim, len(tokens)
        half = hd // 2
        inv = m.position.theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / hd)
        ang = torch.outer(torch.arange(t, dtype=torch.float64), inv)
        cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]

        def norm(x, g, eps):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g

        def rope(x):
            a, b = x[..., :half], x[..., half:]
            return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
        x = weights["emb"][torch.tensor(tokens)]
        causal = torch.full((t, t), float("-inf")).triu(1)
        for w in weights["layers"]:
            n = norm(x, w["n1"], layer0.mixer_norm.eps)
            q = rope((n @ w["q"].T).view(t, hq, hd))
            k = rope((n @ w["k"].T).view(t, hkv, hd)).repeat_interleave(hq // hkv, dim=1)
            v = (n @ w["v"].T).view(t, hkv, hd).repeat_interleave(hq // hkv, dim=1)
            sc = torch.einsum("thd,shd->hts", q, k) / math.sqrt(hd) + causal
            a = torch.einsum("hts,shd->thd", torch.softmax(sc, dim=-1), v).reshape(t, hq * hd)
            x = x + a @ w["o"].T
            n = norm(x, w["n2"], layer0.feed_forward_norm.eps)
            g = n @ w["gate"].T
            x = x + ((g / (1 + torch.exp(-g))) * (n @ w["up"].T)) @ w["down"].T
        x = norm(x, weights["norm"], cfg.final_norm.eps)
        return x @ (weights["emb"] if cfg.tie_word_embeddings else weights["head"]).T

    def random_weights(cfg):
        layer0 = cfg.layers[0]
        m, f, d = layer0.mixer, layer0.feed_forward, cfg.hidden_size
        r = lambda *s_: torch.randn(*s_) * 0.02
        layers = [dict(n1=torch.ones(d), n2=torch.ones(d), q=r(m.n_heads * m.head_dim, d),
                       k=r(m.n_kv_heads * m.head_dim, d), v=r(m.n_kv_heads * m.head_dim, d),
                       o=r(d, m.n_heads * m.head_dim), gate=r(f.intermediate, d),
                       up=r(f.intermediate, d), down=r(d, f.intermediate))
                  for _ in range(len(cfg.layers))]
        return dict(emb=r(cfg.vocab_size, d), head=r(cfg.vocab_size, d), norm=torch.ones(d),
                    layers=layers)

    out = {}
    for name, t, layers in (("tiny-a", 64, None), ("tiny-b", 130, None), ("120m", 128, 1)):
        raw = shape(name)
        if layers:
            raw["n_layer"] = layers
        cfg = parse_config(raw)
        weights = random_weights(cfg)
        tokens = [(7 * i + 3) % cfg.vocab_size for i in range(t)]
        forward(cfg, weights, tokens)
        reps = 5
        t0 = time.perf_counter()
        for _ in range(reps):
            forward(cfg, weights, tokens)
        dt = (time.perf_counter() - t0) / reps
        out[f"{name}_tokens_per_s"] = round(t / dt, 1)
        out[f"{name}_tokens"] = t
        out[f"{name}_layers"] = len(cfg.layers)
    out["threads"] = torch.get_num_threads()
    out["what"] = "plain float32 forward of a whole sequence on the CPU, no cache"
    print(json.dumps({"impl": "cpu", "metric": "plain CPU forward, tokens/s", "dtype": "fp32",
                      "data": "synthetic", "cpu_baseline": out}))
    return 0


def run_profile_case(args):
    """A small workload for a profiler (ncu): builds the 120M shape with
    `--layers` layers, fills `--batch` requests to `--context` tokens, then runs
    `--steps` eager steps of the named kind between cudaProfilerStart and
    cudaProfilerStop, so that `ncu --profile-from-start off` sees only those."""
    import torch
    from crucible_b200 import LLM, ops
    from crucible_b200.config import shape
    from crucible_b200.engine import StepEntry
    from crucible_b200.weights import write_random_model
    raw = shape(args.shape)
    if args.layers:
        raw["n_layer" if "n_layer" in raw else "num_hidden_layers"] = args.layers
    rng = random.Random(1)
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(raw, os.path.join(tmp, "model"), seed=0)
        pages = 64 * (-(-(args.context + args.steps + 64) // 16)) + 64
        llm = LLM(folder, dtype="bfloat16", max_batch=64, kv_pages=pages, prefill_token_budget=2048,
                  graph=False)
    engine = llm.engine
    vocab = engine.config.vocab_size
    if args.profile_case == "prefill":
        n = args.context                                    # one prompt of this many tokens
        tokens = [rng.randrange(vocab) for _ in range(n)]
        engine.step([StepEntry("w", tokens, [n - 1])])
        engine.finish("w")
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for i in range(args.steps):
            engine.step([StepEntry("p", tokens, [n - 1])])
            engine.finish("p")
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    else:
        ids = [f"d{i}" for i in range(args.batch)]
        for rid in ids:
            engine.step([StepEntry(rid, [rng.randrange(vocab) for _ in range(args.context - 1)], [])])
        chosen = torch.zeros(args.batch, dtype=torch.int32, device=engine.device)
        entries = [StepEntry(rid, [0], [0]) for rid in ids]
        for _ in range(2):
            ops.argmax_rows(engine.step(entries, token_source=chosen), chosen)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(args.steps):
            ops.argmax_rows(engine.step(entries, token_source=chosen), chosen)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    print(f"profile case {args.profile_case}: {args.steps} steps, batch {args.batch}, "
          f"{engine.config.n_layers} layers")
    return 0


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=256)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "cpu"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--shape", default="120m", choices=sorted(SHAPE_LABEL),
                   help="a named shape; the default is the benchmark's")
    p.add_argument("--layers", type=int, default=0,
                   help="fewer layers than the shape has (both numbers are reported)")
    p.add_argument("--profile-case", default=None, choices=["prefill", "decode"],
                   help="run a small eager workload for a profiler instead of the benchmark")
    args = p.parse_args()
    if args.profile_case:
        return run_profile_case(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "cpu":
        return run_cpu_baseline(args)
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
