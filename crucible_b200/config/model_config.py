"""Typed model configuration.

A `ModelConfig` is the parsed, validated form of a model folder's config.json.
It is not a bag of Llama numbers: it is a list of `LayerSpec`s (one per stored
layer, each naming its mixer, feed-forward, norms and arrangement with their
own sizes) plus a run order (which stored layer runs when, and whose cache it
reads).  Architectures translate their own config.json spelling into this form
(see `crucible_b200/models/`); everything below the registry reads only this.

Reference behaviour this mirrors: `engine/src/config.rs:13-38` (keys),
`engine/src/config.rs:61-91` (validation: divisibility, enumerated strings),
`engine/src/config.rs:93-105` (derived head_dim, n_rep).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be executed; the message names the key."""


@dataclass(frozen=True)
class NormSpec:
    kind: str              # registered norm kind, e.g. "rmsnorm"
    width: int
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    kind: str              # registered position encoding, e.g. "rope"
    rotary_dim: int        # how many leading features of a head are rotated
    theta: float
    max_positions: int


@dataclass(frozen=True)
class MixerSpec:
    kind: str              # registered mixer kind, e.g. "attention"
    width: int             # model width it reads and writes
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    softmax_scale: float = 0.0
    window: Optional[int] = None      # None = all earlier keys
    position: Optional[PositionSpec] = None
    extra: Tuple[Tuple[str, Any], ...] = ()   # free-form options for other kinds

    def option(self, key: str, default: Any = None) -> Any:
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str              # registered feed-forward kind, e.g. "swiglu"
    width: int
    intermediate: int
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One stored layer.  `norms` are the arrangement's norms by name, as many as it
    asks for: two for `pre_norm` ("mixer_norm", "feed_forward_norm"); an arrangement
    with sandwich norms or with one norm for parallel branches names others.  The names
    are also the parts' paths ("layer.<name>.gain") in the architecture's tensor names."""
    arrangement: str       # registered block arrangement, e.g. "pre_norm"
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    norms: Tuple[Tuple[str, NormSpec], ...]

    def norm(self, name: str) -> NormSpec:
        for key, spec in self.norms:
            if key == name:
                return spec
        raise ConfigError(f"the layer has no norm named {name!r} "
                          f"(it has {[k for k, _ in self.norms]})")

    @property
    def mixer_norm(self) -> NormSpec:
        return self.norm("mixer_norm")

    @property
    def feed_forward_norm(self) -> NormSpec:
        return self.norm("feed_forward_norm")


def pre_norm_layer(mixer: MixerSpec, mixer_norm: NormSpec, feed_forward: FeedForwardSpec,
                   feed_forward_norm: NormSpec) -> LayerSpec:
    """x += mixer(norm(x)); x += feed_forward(norm(x))."""
    return LayerSpec(arrangement="pre_norm", mixer=mixer, feed_forward=feed_forward,
                     norms=(("mixer_norm", mixer_norm), ("feed_forward_norm", feed_forward_norm)))


@dataclass(frozen=True)
class EndSpec:
    """The token embedding or the LM head: a registered kind and free-form options
    (an embedding scale, a soft cap of the logits, a bias: whatever that kind reads)."""
    kind: str
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run stored layer `layer`; if `cache_of` is
    set, its mixer reads (and does not write) the cache that layer owns."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_context: int
    tie_word_embeddings: bool
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: NormSpec
    embedding: EndSpec = EndSpec("token")
    head: EndSpec = EndSpec("linear")
    tensor_names: Mapping[str, str] = field(default_factory=dict, compare=False)
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def validate(self) -> "ModelConfig":
        _positive("vocab_size", self.vocab_size)
        _positive("hidden_size", self.hidden_size)
        _positive("max_context", self.max_context)
        if not self.layers:
            raise ConfigError("the model has no layers")
        for i, entry in enumerate(self.run_order):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"run_order[{i}] names layer {entry.layer}, "
                                  f"but there are {len(self.layers)} layers")
            if entry.cache_of is not None and not 0 <= entry.cache_of < len(self.layers):
                raise ConfigError(f"run_order[{i}] reads the cache of layer "
                                  f"{entry.cache_of}, which does not exist")
        for i, layer in enumerate(self.layers):
            names = [name for name, _ in layer.norms]
            if len(set(names)) != len(names):
                raise ConfigError(f"layer {i} names a norm twice: {names}")
            for what, width in ([("mixer", layer.mixer.width),
                                 ("feed_forward", layer.feed_forward.width)]
                                + [(name, spec.width) for name, spec in layer.norms]):
                if width != self.hidden_size:
                    raise ConfigError(f"layer {i} {what} width {width} differs from "
                                      f"hidden_size {self.hidden_size}")
        return self


def _positive(key: str, value: Any) -> None:
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{key} must be a positive integer, got {value!r}")


# ---------------------------------------------------------------------------
# Helpers shared by architecture parsers
# ---------------------------------------------------------------------------

class KeyReader:
    """Reads keys of a config.json dict with typed errors that name the key."""

    def __init__(self, raw: Mapping[str, Any], where: str = "config.json"):
        self.raw = raw
        self.where = where

    def has(self, key: str) -> bool:
        return key in self.raw and self.raw[key] is not None

    def integer(self, key: str, default: Optional[int] = None) -> int:
        if not self.has(key):
            if default is None:
                raise ConfigError(f"{self.where}: required key {key!r} is missing")
            return default
        v = self.raw[key]
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: {key!r} must be an integer, got {v!r}")
        if v <= 0:
            raise ConfigError(f"{self.where}: {key!r} must be positive, got {v}")
        return v

    def number(self, key: str, default: Optional[float] = None) -> float:
        if not self.has(key):
            if default is None:
                raise ConfigError(f"{self.where}: required key {key!r} is missing")
            return float(default)
        v = self.raw[key]
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: {key!r} must be a number, got {v!r}")
        v = float(v)
        if not math.isfinite(v) or v <= 0.0:
            raise ConfigError(f"{self.where}: {key!r} must be a positive finite number, got {v}")
        return v

    def boolean(self, key: str, default: bool) -> bool:
        if not self.has(key):
            return default
        v = self.raw[key]
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: {key!r} must be true or false, got {v!r}")
        return v

    def choice(self, key: str, allowed: Tuple[str, ...], default: Optional[str] = None) -> str:
        if not self.has(key):
            if default is None:
                raise ConfigError(f"{self.where}: required key {key!r} is missing")
            return default
        v = self.raw[key]
        if v not in allowed:
            raise ConfigError(f"{self.where}: unsupported {key}: {v!r} "
                              f"(this engine runs {list(allowed)})")
        return v


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir}")
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}")
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw
