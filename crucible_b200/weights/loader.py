"""Loading a model's tensors by name, with one error that lists every problem.

The reference reads each tensor by name and fails at the first missing one
(`engine/src/weights.rs:54-94`); its exporter checks missing and unexpected
keys together (`export.py:79-83`).  Here all problems of a checkpoint are
gathered first: missing tensors, unexpected tensors, wrong shapes, unusable
dtypes -- and reported in one `WeightError`.

Dtype rule.  Matrices (operands of matrix products, gathered tables) are kept
in the engine dtype: bfloat16 for the bfloat16 engine (a matrix stored in
32 bits is rounded to nearest-even once, at load), float32 for the float32
engine (bfloat16 and float16 widen exactly).  Vectors (gains and the like) are
kept in float32 in both engines, so a vector stored in 32 bits stays so.
Integer tables are kept as int32.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """A checkpoint that does not fit the model; lists every problem found."""

    def __init__(self, path, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"{path} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the model needs {list(want)}")
        for name, got, role in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, which cannot be a {role}")
        super().__init__("\n".join(lines))


def load_weights(model, model_dir: str, dtype: torch.dtype, device) -> None:
    """Reads model.safetensors of `model_dir` into `model` (a DecoderModel)."""
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"engine dtype must be bfloat16 or float32, got {dtype}")
    path = os.path.join(model_dir, "model.safetensors")
    try:
        f = SafetensorsFile(path)
    except SafetensorsError as e:
        raise WeightError(path, [str(e)], [], [], []) from None
    try:
        requests = model.tensor_requests()
        wanted = {r.checkpoint_name for r in requests}
        missing, wrong_shape, wrong_dtype = [], [], []
        for r in requests:
            if r.checkpoint_name not in f:
                if not r.decl.optional:
                    missing.append(r.checkpoint_name)
                continue
            e = f.entries[r.checkpoint_name]
            if tuple(e.shape) != tuple(r.decl.shape):
                wrong_shape.append((r.checkpoint_name, e.shape, r.decl.shape))
            stored = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16}.get(e.dtype)
            if r.decl.role == "int_table":
                if e.dtype not in ("I64", "I32", "I16", "I8", "U8"):
                    wrong_dtype.append((r.checkpoint_name, e.dtype, "integer table"))
            elif stored is None:
                wrong_dtype.append((r.checkpoint_name, e.dtype, r.decl.role))
        unexpected = sorted(n for n in f.names() if n not in wanted)
        # A tied model's checkpoint may still carry the head's copy of the
        # table; the reference's exporter drops it (`export.py:68-69`) but a
        # file that keeps it holds nothing the model lacks.
        tolerated = set()
        if model.config.tie_word_embeddings:
            head_name = model.config.tensor_names.get("head.weight")
            if head_name in unexpected:
                tolerated.add(head_name)
        unexpected = [n for n in unexpected if n not in tolerated]
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightError(path, missing, unexpected, wrong_shape, wrong_dtype)
        loaded: Dict[str, Optional[torch.Tensor]] = {}
        for r in requests:
            if r.checkpoint_name not in f:
                loaded[r.key] = None
                continue
            t = f.get(r.checkpoint_name)
            if r.decl.role == "matrix":
                t = t.to(dtype)
            elif r.decl.role == "vector":
                t = t.to(torch.float32)
            else:
                t = t.to(torch.int32)
            loaded[r.key] = t.contiguous().to(device)
    finally:
        f.close()
    model.bind(loaded, dtype, torch.device(device))
