"""Each part of a layer alone against its plain function, and toy parts defined
here (a mixer with state of its own, a feed-forward with routing, a position
encoding that is not a rotation, a run order that names a layer twice and reads
another layer's cache) registered, built and stepped without a change to the
framework's files."""
import math
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel(got, ref):
    return float((got.double().cpu() - ref.double()).abs().max()) / max(float(ref.abs().max()), 1e-6)


def _ctx(n_tokens, positions=None, dtype=torch.float32):
    """A minimal step context for parts that need no cache."""
    from crucible_b200.engine.context import Scratch
    scratch = Scratch(torch.device(DEV))
    pos = positions if positions is not None else list(range(n_tokens))
    return SimpleNamespace(scratch=scratch.get, n_tokens=n_tokens, dtype=dtype,
                           positions=torch.tensor(pos, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 5e-3)])
def test_norm_part(dtype, tol):
    from crucible_b200.config import NormSpec
    from crucible_b200.parts import NORMS
    norm = NORMS.build("rmsnorm", NormSpec("rmsnorm", 200, 3e-4))
    assert [(d.name, d.shape, d.role) for d in norm.tensors()] == [("gain", (200,), "vector")]
    gain = 1 + 0.3 * torch.randn(200)
    norm.bind({"gain": gain.to(DEV)}, dtype, torch.device(DEV))
    x = torch.randn(13, 200) * 2
    out = norm.forward(_ctx(13), x.to(DEV))
    assert out.dtype == dtype
    assert rel(out, pm.plain_rmsnorm(x.double(), gain.double(), 3e-4)) < tol


def test_position_part_tables():
    from crucible_b200.config import PositionSpec
    from crucible_b200.parts import POSITIONS
    rope = POSITIONS.build("rope", PositionSpec("rope", 24, 777.0, 50))
    rope.bind({}, torch.float32, torch.device(DEV))
    cos, sin, dim = rope.rotation()
    want_cos, want_sin = pm.plain_rope_tables(24, 50, 777.0)
    assert dim == 24 and cos.shape == (50, 12)
    assert rel(cos, want_cos) < 1e-7 and rel(sin, want_sin) < 1e-7


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
def test_feed_forward_part(dtype, tol):
    from crucible_b200.config import FeedForwardSpec
    from crucible_b200.parts import FEED_FORWARDS
    ffn = FEED_FORWARDS.build("swiglu", FeedForwardSpec("swiglu", 72, 200))
    assert sorted(d.name for d in ffn.tensors()) == ["down", "gate", "up"]
    w = {k: (torch.randn(s) * 0.2).bfloat16() for k, s in
         (("gate", (200, 72)), ("up", (200, 72)), ("down", (72, 200)))}
    ffn.bind({k: v.to(dtype).to(DEV) for k, v in w.items()}, dtype, torch.device(DEV))
    h = torch.randn(9, 72).bfloat16()
    residual = torch.randn(9, 72)
    res_dev = residual.clone().to(DEV)
    ffn.forward(_ctx(9), h.to(dtype).to(DEV), res_dev)
    want = residual.double() + pm.plain_swiglu(h.double(), w["gate"].double(), w["up"].double(),
                                               w["down"].double())
    assert rel(res_dev, want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_and_block_through_the_engine(tmp_path, dtype):
    """The mixer and the block arrangement with real cache bindings: a one-layer
    model's residual stream after the block, read back from the engine's scratch."""
    name = "tiny-b"
    raw = dict(helpers.TINY[name]["config"], num_hidden_layers=1)
    from crucible_b200.weights import write_random_model
    from crucible_b200.engine import Engine, EngineOptions, StepEntry
    folder = write_random_model(raw, str(tmp_path / "one"), seed=4, std=helpers.TEST_STD)
    eng = Engine(folder, EngineOptions(dtype=dtype, page_tokens=32, n_pages=4, max_requests=1))
    tokens = helpers.random_tokens(raw["vocab_size"], 70, 5)
    eng.step([StepEntry("a", tokens[:41], [])])
    eng.step([StepEntry("a", tokens[41:], [28])])
    x = eng.scratch.get("residual", (29, raw["hidden_size"]), torch.float32).cpu()
    cfg, w = pm.read_folder(folder)
    cos, sin = pm.plain_rope_tables(cfg["head_dim"], 70, cfg["theta"])
    want = pm.plain_block(pm.plain_embedding(w[pm.tensor_name(cfg, "embed")], tokens), cfg, w, 0,
                          cos, sin)[41:]
    assert rel(x, want) < (1e-5 if dtype == "float32" else 2e-2)


# ---------------------------------------------------------------------------
# toy parts, defined here
# ---------------------------------------------------------------------------

WIDTH, HEADS, KV, HD, INTER, VOCAB = 32, 2, 1, 16, 48, 61
DECAY = 0.75


def _register_toys():
    from crucible_b200.config import (Architecture, FeedForwardSpec, MixerSpec, ModelConfig, NormSpec,
                                      PositionSpec, RunEntry, pre_norm_layer, register_architecture)
    from crucible_b200.config.registry import _ARCHITECTURES
    from crucible_b200.parts import (FEED_FORWARDS, MIXERS, POSITIONS, FeedForward, Mixer,
                                     PositionEncoding, TensorDecl)

    class EmaMixer(Mixer):
        """State of fixed size per request: s = decay * s + (1 - decay) * h, y = s W^T."""
        graph_safe_prompt_steps = False      # portions are walked in a host loop below

        def __init__(self, spec):
            self.spec = spec
            self.decay = float(spec.option("decay"))

        def tensors(self):
            return [TensorDecl("mix", (self.spec.width, self.spec.width))]

        def bind(self, tensors, dtype, device):
            self.mix = tensors["mix"].float()

        def state_bytes(self):
            return 4 * self.spec.width

        def forward(self, ctx, h, residual, binding):
            state = ctx.state(binding).view(torch.float32)          # [slots, width]
            slots = ctx.req_state_slot.long()
            if ctx.host.all_single_token:                          # device-side only: replayable
                s = state.index_select(0, slots) * self.decay + h.float() * (1 - self.decay)
                state.index_copy_(0, slots, s)
                residual.add_(s @ self.mix.T)
                return
            row = 0
            for r, n in enumerate(ctx.host.new_tokens):
                s = state[ctx.host.state_slots[r]].clone()
                for i in range(n):
                    s = s * self.decay + h[row + i].float() * (1 - self.decay)
                    residual[row + i] += s @ self.mix.T
                state[ctx.host.state_slots[r]] = s
                row += n

    class RoutedFeedForward(FeedForward):
        """Two experts, router logits in fp32, the better expert per row (ties to the lower)."""
        def __init__(self, spec):
            self.spec = spec

        def tensors(self):
            d, i = self.spec.width, self.spec.intermediate
            return [TensorDecl("router", (2, d)), TensorDecl("up", (2 * i, d)),
                    TensorDecl("down", (2 * d, i))]

        def bind(self, tensors, dtype, device):
            self.router = tensors["router"].float()
            self.up = tensors["up"].float()
            self.down = tensors["down"].float()

        def forward(self, ctx, h, residual):
            d, i = self.spec.width, self.spec.intermediate
            hf = h.float()
            choice = (hf @ self.router.T).argmax(dim=-1)
            outs = [torch.relu(hf @ self.up[e * i:(e + 1) * i].T) @ self.down[e * d:(e + 1) * d].T
                    for e in range(2)]
            residual.add_(torch.where(choice.unsqueeze(1) == 0, outs[0], outs[1]))

    class AdditivePosition(PositionEncoding):
        """Not a rotation: adds sin(position * (feature + 1) * step) to q and k."""
        def __init__(self, spec):
            self.spec = spec

        def bind(self, tensors, dtype, device):
            pos = torch.arange(self.spec.max_positions, dtype=torch.float64).unsqueeze(1)
            feat = torch.arange(1, self.spec.rotary_dim + 1, dtype=torch.float64).unsqueeze(0)
            self.table = torch.sin(pos * feat / self.spec.theta).float().to(device)

        def apply(self, ctx, q, k):
            add = self.table.index_select(0, ctx.positions.long()).unsqueeze(1)
            q.add_(add.to(q.dtype))
            k.add_(add.to(k.dtype))

    for reg, kind, maker in ((MIXERS, "ema", EmaMixer), (FEED_FORWARDS, "routed", RoutedFeedForward),
                             (POSITIONS, "additive", AdditivePosition)):
        reg.register(kind, maker, replace=True)

    names = {
        "embedding.table": "emb", "head.weight": "head", "final_norm.gain": "norm",
        "layer.mixer_norm.gain": "l{layer}.n1", "layer.feed_forward_norm.gain": "l{layer}.n2",
        "layer.mixer.q": "l{layer}.q", "layer.mixer.k": "l{layer}.k", "layer.mixer.v": "l{layer}.v",
        "layer.mixer.o": "l{layer}.o", "layer.mixer.mix": "l{layer}.mix",
        "layer.feed_forward.gate": "l{layer}.gate", "layer.feed_forward.up": "l{layer}.up",
        "layer.feed_forward.down": "l{layer}.down", "layer.feed_forward.router": "l{layer}.router",
    }

    def parse(raw):
        norm = NormSpec("rmsnorm", WIDTH, raw["eps"])
        attn = MixerSpec("attention", WIDTH, HEADS, KV, HD, 1 / math.sqrt(HD), None,
                         PositionSpec("additive", HD, raw["step"], raw["ctx"]))
        ema = MixerSpec("ema", WIDTH, extra=(("decay", raw["decay"]),))
        layers = (pre_norm_layer(attn, norm, FeedForwardSpec("swiglu", WIDTH, INTER), norm),
                  pre_norm_layer(ema, norm, FeedForwardSpec("routed", WIDTH, INTER), norm))
        # layer 0 runs twice; its second run reads the cache the first one wrote
        order = (RunEntry(0), RunEntry(1), RunEntry(0, cache_of=0))
        return ModelConfig("ToyHybrid", VOCAB, WIDTH, raw["ctx"], False, layers, order, norm,
                           tensor_names=names, raw=dict(raw))

    _ARCHITECTURES.pop("ToyHybrid", None)
    register_architecture(Architecture("ToyHybrid", parse, lambda cfg: dict(cfg.raw)))
    return {"architectures": ["ToyHybrid"], "eps": 1e-5, "step": 7.0, "ctx": 96, "decay": DECAY}


def _toy_oracle(w, tokens, raw):
    """The toy model on a whole sequence, plainly."""
    t = len(tokens)
    x = w["emb"][torch.tensor(tokens)]
    pos = torch.arange(t, dtype=torch.float64).unsqueeze(1)
    feat = torch.arange(1, HD + 1, dtype=torch.float64).unsqueeze(0)
    add = torch.sin(pos * feat / raw["step"]).float().double().unsqueeze(1)

    def attention_layer(x, kv=None):
        n = pm.plain_rmsnorm(x, w["l0.n1"], raw["eps"])
        q = (n @ w["l0.q"].T).view(t, HEADS, HD) + add
        if kv is None:
            k = (n @ w["l0.k"].T).view(t, KV, HD) + add
            v = (n @ w["l0.v"].T).view(t, KV, HD)
            kv = (k, v)
        x = x + pm.plain_attention(q, kv[0], kv[1]).reshape(t, HEADS * HD) @ w["l0.o"].T
        n = pm.plain_rmsnorm(x, w["l0.n2"], raw["eps"])
        return x + pm.plain_swiglu(n, w["l0.gate"], w["l0.up"], w["l0.down"]), kv

    x, kv = attention_layer(x)
    n = pm.plain_rmsnorm(x, w["l1.n1"], raw["eps"])
    s = torch.zeros(WIDTH, dtype=torch.float64)
    ys = []
    for i in range(t):
        s = s * DECAY + n[i] * (1 - DECAY)
        ys.append(s @ w["l1.mix"].T)
    x = x + torch.stack(ys)
    n = pm.plain_rmsnorm(x, w["l1.n2"], raw["eps"])
    choice = (n @ w["l1.router"].T).argmax(dim=-1)
    outs = [torch.relu(n @ w["l1.up"][e * INTER:(e + 1) * INTER].T) @ w["l1.down"][e * WIDTH:(e + 1) * WIDTH].T
            for e in range(2)]
    x = x + torch.where(choice.unsqueeze(1) == 0, outs[0], outs[1])
    x, _ = attention_layer(x, kv)
    return pm.plain_rmsnorm(x, w["norm"], raw["eps"]) @ w["head"].T


def test_toy_parts_are_registered_built_and_stepped(tmp_path):
    from crucible_b200.engine import Engine, EngineOptions, StepEntry
    from crucible_b200.weights import write_random_model
    from safetensors import safe_open
    raw = _register_toys()
    folder = write_random_model(raw, str(tmp_path / "toy"), seed=9, std=0.15)
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        w = {k: f.get_tensor(k).double() for k in f.keys()}
    eng = Engine(folder, EngineOptions(dtype="float32", page_tokens=16, n_pages=12, max_requests=3))
    assert len(eng.model.cache_groups) == 1 and eng.model.cache_groups[0].layers == (0,)
    assert eng.model.state_bytes == 4 * WIDTH
    assert [b.write for b in eng.model.bindings] == [True, True, False]
    seqs = {"a": helpers.random_tokens(VOCAB, 50, 1), "b": helpers.random_tokens(VOCAB, 37, 2)}
    refs = {k: _toy_oracle(w, v, raw).numpy() for k, v in seqs.items()}
    got = {}

    def run(entries):
        logits = eng.step([StepEntry(r, t, want) for r, t, want in entries]).cpu().numpy()
        i = 0
        for r, t, want in entries:
            start = eng.held_tokens(r) - len(t)
            for wpos in want:
                got[(r, start + wpos)] = logits[i]
                i += 1
    # portions of a beside b; then both one token at a time (captured and replayed)
    run([("a", seqs["a"][:20], [0, 19])])
    run([("a", seqs["a"][20:33], [12]), ("b", seqs["b"][:30], [29])])
    run([("a", seqs["a"][33:40], list(range(7))), ("b", seqs["b"][30:32], [0, 1])])
    for i in range(5):
        run([("a", [seqs["a"][40 + i]], [0]), ("b", [seqs["b"][32 + i]], [0])])
    for i in range(5):
        run([("a", [seqs["a"][45 + i]], [0])])
    assert eng._graphs and not eng._graph_failed, eng._graph_error
    for (r, pos), row in got.items():
        assert helpers.relative_error(row, refs[r][pos]) < 3e-5, (r, pos)
    # a new request gets a clean state slot after the old ones are gone
    eng.finish("a"); eng.finish("b")
    run([("c", seqs["b"][:10], [9])])
    assert helpers.relative_error(got[("c", 9)], refs["b"][9]) < 3e-5


def test_model_layouts_are_checked():
    from crucible_b200.config import (ConfigError, ModelConfig, RunEntry, parse_config)
    from crucible_b200.models.decoder import DecoderModel
    raw = _register_toys()
    cfg = parse_config(raw)
    import dataclasses
    bad = dataclasses.replace(cfg, run_order=(RunEntry(0), RunEntry(0)))
    with pytest.raises(ConfigError, match="second time"):
        DecoderModel(bad)
    bad = dataclasses.replace(cfg, run_order=(RunEntry(1), RunEntry(0, cache_of=1)))
    with pytest.raises(ConfigError, match="keeps none"):
        DecoderModel(bad)
    bad = dataclasses.replace(cfg, run_order=(RunEntry(1, cache_of=0), RunEntry(0)))
    with pytest.raises(ConfigError):
        DecoderModel(bad)


# ---------------------------------------------------------------------------
# a window: pages given back while the request runs, through the whole engine
# ---------------------------------------------------------------------------

WINDOW = 40


def _register_windowed():
    """The dense decoder with a window on every layer's attention: the reference's own
    keys plus "window".  Defined here; the framework's files know nothing of it."""
    import dataclasses
    from crucible_b200.config import Architecture, register_architecture
    from crucible_b200.config.registry import _ARCHITECTURES
    from crucible_b200.models import crucible_gpt

    def parse(raw):
        base = crucible_gpt._parse_crucible({k: v for k, v in raw.items() if k != "window"})
        layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, window=raw["window"]))
                       for l in base.layers)
        return dataclasses.replace(base, architecture="WindowedGPT", layers=layers, raw=dict(raw))

    _ARCHITECTURES.pop("WindowedGPT", None)
    register_architecture(Architecture("WindowedGPT", parse, lambda cfg: dict(cfg.raw)))
    return {"architectures": ["WindowedGPT"], "vocab_size": 211, "n_layer": 2, "n_head": 4,
            "n_kv_head": 2, "n_embd": 96, "head_dim": 48, "intermediate_size": 160,
            "block_size": 384, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": True, "window": WINDOW}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_attention_gives_pages_back_and_stays_right(tmp_path, dtype):
    """Window 40, pages of 16, heads of 48 (the mma.sync kernels in bfloat16): portions
    of 20 to 60 tokens, then decoding across several pages that the window has passed
    and the cache manager has given back.  Their table entries name the null page, and
    every page that is free is filled with NaN after each step, so a kernel that read
    a released page (or one it was never given) would show it."""
    from crucible_b200.engine import Engine, EngineOptions, StepEntry
    from crucible_b200.weights import write_random_model
    raw = _register_windowed()
    folder = write_random_model(raw, str(tmp_path / "windowed"), seed=12, std=helpers.TEST_STD)
    cfg, w = pm.read_folder(folder)
    cfg["window"] = WINDOW
    seqs = {"a": helpers.random_tokens(211, 300, 31), "b": helpers.random_tokens(211, 130, 32)}
    refs = {k: pm.plain_forward(cfg, w, v).numpy() for k, v in seqs.items()}
    # 14 pages = 224 tokens for 430 tokens of requests: only a window's worth is ever held
    eng = Engine(folder, EngineOptions(dtype=dtype, page_tokens=16, n_pages=14, max_requests=2))
    assert eng.model.cache_groups[0].need.window == WINDOW
    got, fed = {}, {"a": 0, "b": 0}
    least_free = [14]

    def run(entries):
        batch = []
        for r, n, want in entries:
            batch.append(StepEntry(r, seqs[r][fed[r]:fed[r] + n], want))
        logits = eng.step(batch).float().cpu().numpy()
        i = 0
        for r, n, want in entries:
            for wpos in want:
                got[(r, fed[r] + wpos)] = logits[i]
                i += 1
            fed[r] += n
        eng.cache.check_invariants()
        pool = eng.cache.pools[0]
        least_free[0] = min(least_free[0], pool.free_pages)
        free = [p for p in range(pool.n_pages) if not pool.is_in_use(p)]
        if free:
            eng.storages[0].kv[:, :, free] = float("nan")

    for n in (37, 60, 20, 45, 23):                              # a: 185 tokens in portions
        run([("a", n, [0, n // 2, n - 1])])
    assert eng.cache.held_pages("a", 0) < -(-185 // 16), "no page was given back"
    run([("a", 1, [0]), ("b", 52, [51])])                       # b starts beside a's decoding
    run([("a", 1, [0]), ("b", 33, [0, 32])])
    for _ in range(45):                                         # both decode, crossing pages
        run([("a", 1, [0]), ("b", 1, [0])])
    eng.finish("b")
    while fed["a"] < 300:
        run([("a", 1, [0])])
    assert least_free[0] < 14 - 2 * 3                           # both held their windows at once
    tol = helpers.TOLERANCE[dtype]
    for (r, pos), row in sorted(got.items()):
        assert np.isfinite(row).all(), (r, pos)
        err = helpers.relative_error(row, refs[r][pos])
        assert err <= tol, f"{r} position {pos}: relative error {err:.3g}"
    assert len(got) > 150


# ---------------------------------------------------------------------------
# another arrangement and other ends, defined here
# ---------------------------------------------------------------------------

def test_sandwich_norms_scaled_embedding_and_capped_head_without_framework_edits(tmp_path):
    """An arrangement with four norms (before and after each branch), an embedding that
    scales its rows and a head that soft-caps its logits: registered here, named by a toy
    architecture's config, built and stepped by the unchanged framework."""
    from crucible_b200 import ops
    from crucible_b200.config import (Architecture, EndSpec, FeedForwardSpec, LayerSpec, MixerSpec,
                                      ModelConfig, NormSpec, PositionSpec, RunEntry,
                                      register_architecture)
    from crucible_b200.config.registry import _ARCHITECTURES
    from crucible_b200.engine import Engine, EngineOptions, StepEntry
    from crucible_b200.parts import (ARRANGEMENTS, EMBEDDINGS, HEADS, Arrangement, Embedding, Head,
                                     TensorDecl)
    from crucible_b200.weights import write_random_model
    from safetensors import safe_open
    width, heads, kv, hd, inter, vocab, eps, cap, scale = 48, 3, 1, 16, 80, 97, 1e-5, 3.0, 1.7

    class Sandwich(Arrangement):
        norm_names = ("pre_mixer", "post_mixer", "pre_ffn", "post_ffn")

        def forward(self, ctx, x, binding):
            for pre, post, branch, extra in (("pre_mixer", "post_mixer", self.mixer, (binding,)),
                                             ("pre_ffn", "post_ffn", self.feed_forward, ())):
                h = self.norms[pre].forward(ctx, x)
                y = torch.zeros_like(x)                      # the branch's output alone
                branch.forward(ctx, h, y, *extra)
                x.add_(self.norms[post].forward(ctx, y).float())

    class ScaledEmbedding(Embedding):
        def __init__(self, spec, vocab_size, w):
            self.vocab_size, self.width, self.scale = vocab_size, w, float(spec.option("scale"))

        def tensors(self):
            return [TensorDecl("table", (self.vocab_size, self.width))]

        def bind(self, tensors, dtype, device):
            self.table = tensors["table"]

        def forward(self, ctx, token_ids):
            x = ctx.scratch("residual", (token_ids.shape[0], self.width), torch.float32)
            ops.embed_rows(self.table, token_ids, x, ctx.device_tokens)
            return x.mul_(self.scale)

    class CappedHead(Head):
        def __init__(self, spec, vocab_size, w, tied):
            self.vocab_size, self.cap = vocab_size, float(spec.option("cap"))

        def tie(self, table):
            self.weight = table

        def forward(self, ctx, rows):
            logits = ctx.scratch("logits", (rows.shape[0], self.vocab_size), torch.float32)
            ops.linear(rows, self.weight, logits)
            return logits.copy_(torch.tanh(logits / self.cap) * self.cap)

    ARRANGEMENTS.register("sandwich", Sandwich, replace=True)
    EMBEDDINGS.register("scaled", ScaledEmbedding, replace=True)
    HEADS.register("capped", CappedHead, replace=True)
    names = {"embedding.table": "emb", "final_norm.gain": "norm",
             "layer.pre_mixer.gain": "l{layer}.n0", "layer.post_mixer.gain": "l{layer}.n1",
             "layer.pre_ffn.gain": "l{layer}.n2", "layer.post_ffn.gain": "l{layer}.n3",
             "layer.mixer.q": "l{layer}.q", "layer.mixer.k": "l{layer}.k", "layer.mixer.v": "l{layer}.v",
             "layer.mixer.o": "l{layer}.o", "layer.feed_forward.gate": "l{layer}.gate",
             "layer.feed_forward.up": "l{layer}.up", "layer.feed_forward.down": "l{layer}.down"}

    def parse(raw):
        norm = NormSpec("rmsnorm", width, eps)
        attn = MixerSpec("attention", width, heads, kv, hd, 1 / math.sqrt(hd), None,
                         PositionSpec("rope", hd, 10000.0, raw["ctx"]))
        layer = LayerSpec("sandwich", attn, FeedForwardSpec("swiglu", width, inter),
                          tuple((n, norm) for n in Sandwich.norm_names))
        return ModelConfig("ToySandwich", vocab, width, raw["ctx"], True, (layer, layer),
                           (RunEntry(0), RunEntry(1)), norm,
                           embedding=EndSpec("scaled", (("scale", raw["scale"]),)),
                           head=EndSpec("capped", (("cap", raw["cap"]),)),
                           tensor_names=names, raw=dict(raw))

    _ARCHITECTURES.pop("ToySandwich", None)
    register_architecture(Architecture("ToySandwich", parse, lambda cfg: dict(cfg.raw)))
    raw = {"architectures": ["ToySandwich"], "ctx": 64, "scale": scale, "cap": cap}
    folder = write_random_model(raw, str(tmp_path / "sandwich"), seed=3, std=0.2)
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        w = {k: f.get_tensor(k).double() for k in f.keys()}
    # a layer that asks for norms the arrangement does not have is refused when built
    from crucible_b200.models.decoder import DecoderModel
    import dataclasses
    cfg = parse(raw)
    bad = dataclasses.replace(cfg, layers=(dataclasses.replace(cfg.layers[0], arrangement="pre_norm"),) * 2)
    with pytest.raises(ValueError, match="needs the norms"):
        DecoderModel(bad)

    tokens = helpers.random_tokens(vocab, 40, 8)
    t = len(tokens)
    cos, sin = pm.plain_rope_tables(hd, t, 10000.0)
    x = pm.plain_embedding(w["emb"], tokens) * scale
    for l in range(2):
        n = pm.plain_rmsnorm(x, w[f"l{l}.n0"], eps)
        q = pm.plain_rope((n @ w[f"l{l}.q"].T).view(t, heads, hd), cos, sin)
        k = pm.plain_rope((n @ w[f"l{l}.k"].T).view(t, kv, hd), cos, sin)
        v = (n @ w[f"l{l}.v"].T).view(t, kv, hd)
        y = pm.plain_attention(q, k, v).reshape(t, heads * hd) @ w[f"l{l}.o"].T
        x = x + pm.plain_rmsnorm(y, w[f"l{l}.n1"], eps)
        n = pm.plain_rmsnorm(x, w[f"l{l}.n2"], eps)
        y = pm.plain_swiglu(n, w[f"l{l}.gate"], w[f"l{l}.up"], w[f"l{l}.down"])
        x = x + pm.plain_rmsnorm(y, w[f"l{l}.n3"], eps)
    want = pm.plain_rmsnorm(x, w["norm"], eps) @ w["emb"].T
    want = (torch.tanh(want / cap) * cap).numpy()

    eng = Engine(folder, EngineOptions(dtype="float32", page_tokens=16, n_pages=6, max_requests=1))
    first = eng.step([StepEntry("a", tokens[:23], [0, 22])]).cpu().numpy()
    assert helpers.relative_error(first[0], want[0]) < 3e-5
    assert helpers.relative_error(first[1], want[22]) < 3e-5
    for i in range(23, t):
        row = eng.step([StepEntry("a", [tokens[i]], [0])]).cpu().numpy()[0]
        assert helpers.relative_error(row, want[i]) < 3e-5, i
    assert eng._graph_replays > 0 and not eng._graph_failed, eng._graph_error
