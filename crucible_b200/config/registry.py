"""One registry from an architecture's name to its model.

An `Architecture` knows two things about one model family: how to turn that
family's config.json keys into a `ModelConfig`, and which checkpoint tensor
name each part's tensor has.  Building the model from the `ModelConfig` is the
same generic code for every family (`crucible_b200/models/decoder.py`).

The reference has no registry (one hard-wired model; `engine/src/config.rs:1-6`
"the engine refuses to guess"); the refusal is kept: an unknown architecture
name is an error that lists the known ones.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Any

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Mapping[str, Any]], ModelConfig]
    # Given a ModelConfig, writes back the config.json dict of this family
    # (used by the random-weights mode to emit a loadable folder).
    describe: Callable[[ModelConfig], dict]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    if arch.name in _ARCHITECTURES:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def known_architectures() -> list:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture_name_of(raw: Mapping[str, Any]) -> str:
    """The name a config.json asks for.

    `architectures[0]` (the Hugging Face spelling) or `architecture`; a file
    with neither but with the reference exporter's keys (`export.py:89-97`
    writes `n_embd`, `n_layer`, `pos_encoding`, ... and no name) is the
    reference's own model.
    """
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs:
        return str(archs[0])
    if isinstance(raw.get("architecture"), str):
        return raw["architecture"]
    if "n_embd" in raw and "n_layer" in raw:
        return "CrucibleGPT"
    raise ConfigError("config.json names no architecture (expected "
                      "'architectures': [name] or 'architecture': name)")


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; this engine knows "
                          f"{sorted(_ARCHITECTURES)}") from None


def parse_config(raw: Mapping[str, Any]) -> ModelConfig:
    arch = get_architecture(architecture_name_of(raw))
    return arch.parse(raw).validate()


def load_config(model_dir: str) -> ModelConfig:
    return parse_config(read_config_json(model_dir))


_loaded = False


def _ensure_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from ..models import crucible_gpt  # noqa: F401  (registers on import)
