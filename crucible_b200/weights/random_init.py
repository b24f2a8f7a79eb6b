"""Random-weights mode: writes a model folder from a configuration and a seed.

The folder holds config.json (in the architecture's own spelling) and
model.safetensors with every tensor the model asks for by its checkpoint name.
Matrices are N(0, std) as in the reference's initialiser (`model.py:316-322`,
std 0.02; the 1/sqrt(2L) scaling of residual projections at `model.py:299-304`
is a training device and is not applied); vectors (norm gains) are 1.  Values
are drawn in float32 from a CPU generator seeded per tensor, so the same seed
gives the same folder anywhere, and are stored as bfloat16 (default) or as
float32; with bfloat16 storage both engine dtypes and a plain 32-bit
implementation see exactly the same numbers.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Mapping

import torch

from ..config.registry import get_architecture, parse_config
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(model, seed: int, std: float = 0.02,
                   store_dtype: torch.dtype = torch.bfloat16) -> dict:
    out = {}
    for r in model.tensor_requests():
        if r.decl.role == "vector":
            out[r.checkpoint_name] = torch.ones(r.decl.shape, dtype=torch.float32)
        elif r.decl.role == "int_table":
            out[r.checkpoint_name] = torch.zeros(r.decl.shape, dtype=torch.int32)
        else:
            g = torch.Generator(device="cpu").manual_seed(_tensor_seed(seed, r.checkpoint_name))
            t = torch.randn(r.decl.shape, generator=g, dtype=torch.float32) * std
            out[r.checkpoint_name] = t.to(store_dtype)
    return out


def write_random_model(raw_config: Mapping, out_dir: str, seed: int, *, std: float = 0.02,
                       store_dtype: str = "bfloat16") -> str:
    """Creates `out_dir` with config.json and model.safetensors; returns it."""
    from ..models.decoder import DecoderModel
    if store_dtype not in _STORE:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE)}, got {store_dtype!r}")
    config = parse_config(raw_config)
    model = DecoderModel(config)
    os.makedirs(out_dir, exist_ok=True)
    described = get_architecture(config.architecture).describe(config)
    described["dtype"] = store_dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(described, f, indent=2)
        f.write("\n")
    tensors = random_tensors(model, seed, std, _STORE[store_dtype])
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "source": f"random seed {seed} std {std}"})
    return out_dir
