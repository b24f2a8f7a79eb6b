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
    from crucible_b200.config import (Architecture, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig,
                                      NormSpec, PositionSpec, RunEntry, register_architecture)
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
        layers = (LayerSpec("pre_norm", attn, norm, FeedForwardSpec("swiglu", WIDTH, INTER), norm),
                  LayerSpec("pre_norm", ema, norm, FeedForwardSpec("routed", WIDTH, INTER), norm))
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
