"""Interfaces of the parts a layer is put together from, and their registries.

A layer = a block arrangement over a mixer, a feed-forward and the norms the
arrangement names; a mixer may own a position encoding.  The model's two ends, the
token embedding and the LM head, are registered parts too.  Each kind of part is registered under a name
and built from its spec (sizes and constants are parameters of the spec, never
of the code).  No part knows which model it is in: it sees its spec, its own
tensors under local names, and the `StepContext` of the step being run.

What each interface must provide
--------------------------------
every part
    `tensors()`  -> list of `TensorDecl` (local name, shape, role)
    `bind(tensors, dtype, device)`: receives its loaded tensors (local names)
norm            `forward(ctx, x) -> h`        x: fp32 [T, width] residual stream,
                                              h: [T, width] in the engine dtype
position        `rotation() -> (cos, sin, rotary_dim) | None`, or
                `apply(ctx, q, k)` in place for encodings that are not rotations
mixer           `cache_need() -> CacheNeed | None`, `state_bytes() -> int`,
                `forward(ctx, h, residual, binding)`: residual += mixer(h)
feed-forward    `forward(ctx, h, residual)`: residual += ffn(h)
arrangement     `norm_names`; `forward(ctx, x, binding)`: runs one layer on the residual x
embedding       `forward(ctx, token_ids) -> x`  fp32 [T, width]; `table` if a head may tie to it
head            `forward(ctx, normed_rows) -> logits` fp32 [rows, vocab]; `tie(table)`

The residual stream is always fp32 (the residual sum is a 32-bit sum in both
engine dtypes); `h` and everything a part produces internally is in the engine
dtype (bfloat16 or float32).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

# Roles decide the dtype a tensor is kept in:
#   "matrix": an operand of a matrix product or a gathered table -> engine dtype
#   "vector": gains, biases, per-feature constants -> float32 (a tensor stored
#             in 32 bits stays so; bfloat16 gains are widened exactly)
#   "int_table": integer lookup tables -> int32
ROLES = ("matrix", "vector", "int_table")


@dataclass(frozen=True)
class TensorDecl:
    name: str                      # local name inside the part, e.g. "q"
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False         # absent tensors of optional decls are passed as None


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer needs from the paged cache, per token and per layer."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None   # None: every earlier key stays


@dataclass(frozen=True)
class LayerBinding:
    """Where one run-order entry's mixer keeps what outlives a step: its cache
    group and the layer's slot inside that group's pages (group None: no paged
    cache), whether this run writes them (an entry that reads another layer's
    cache does not), and its byte range inside each request's state slot."""
    group: Optional[int] = None
    slot: int = 0
    write: bool = True
    state_offset: int = 0
    state_bytes: int = 0


class Part:
    # A part whose launches depend only on the step's shape and on device-side
    # metadata can be replayed from a captured CUDA graph.  A part that reads
    # per-step values on the host (other than the shape) sets this to False and
    # the engine then runs every step eagerly.  `graph_safe_prompt_steps` says the same
    # for steps in which some request brings more than one token (a part may, for
    # instance, walk such portions in a host loop but run decode steps from device
    # metadata alone); None means "as graph_safe".
    graph_safe = True
    graph_safe_prompt_steps = None

    def tensors(self) -> List[TensorDecl]:
        return []

    def bind(self, tensors: Dict[str, Optional[torch.Tensor]], dtype: torch.dtype,
             device: torch.device) -> None:
        pass


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotation(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        return None

    def apply(self, ctx, q: torch.Tensor, k: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_bytes(self) -> int:
        return 0

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor,
                binding: LayerBinding) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Arrangement:
    """Puts one layer's parts in order.  Built from the layer's spec and its
    already-built parts; `norm_names` are the norms it needs (the spec must give
    exactly these), `norms` the built ones by name."""
    norm_names: Tuple[str, ...] = ()

    def __init__(self, spec, norms: Dict[str, Norm], mixer: Mixer, feed_forward: FeedForward):
        if set(norms) != set(self.norm_names):
            raise ValueError(f"arrangement {spec.arrangement!r} needs the norms "
                             f"{sorted(self.norm_names)}, the layer gives {sorted(norms)}")
        self.spec = spec
        self.norms = dict(norms)
        self.mixer = mixer
        self.feed_forward = feed_forward

    def forward(self, ctx, x: torch.Tensor, binding: LayerBinding) -> None:
        raise NotImplementedError


class Embedding(Part):
    """Token ids -> rows of the fp32 residual stream."""

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """Normalised rows -> fp32 logits [rows, vocab]; `tie(table)` hands it the
    embedding's table when the model ties them."""

    def tie(self, table: torch.Tensor) -> None:
        raise NotImplementedError

    def forward(self, ctx, normed_rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._makers: Dict[str, Callable] = {}

    def register(self, kind: str, maker: Callable, *, replace: bool = False) -> None:
        if kind in self._makers and not replace:
            raise ValueError(f"{self.what} kind {kind!r} is already registered")
        self._makers[kind] = maker

    def unregister(self, kind: str) -> None:
        self._makers.pop(kind, None)

    def build(self, kind: str, *args, **kwargs):
        try:
            maker = self._makers[kind]
        except KeyError:
            raise ValueError(f"unknown {self.what} kind {kind!r}; registered: "
                             f"{sorted(self._makers)}") from None
        return maker(*args, **kwargs)

    def kinds(self) -> List[str]:
        return sorted(self._makers)


NORMS = _Registry("norm")                   # maker(spec: NormSpec) -> Norm
POSITIONS = _Registry("position encoding")  # maker(spec: PositionSpec) -> PositionEncoding
MIXERS = _Registry("mixer")                 # maker(spec: MixerSpec) -> Mixer
FEED_FORWARDS = _Registry("feed-forward")   # maker(spec: FeedForwardSpec) -> FeedForward
ARRANGEMENTS = _Registry("arrangement")     # maker(spec: LayerSpec, norms: dict, mixer, ffn) -> Arrangement
EMBEDDINGS = _Registry("embedding")         # maker(spec: EndSpec, vocab, width) -> Embedding
HEADS = _Registry("head")                   # maker(spec: EndSpec, vocab, width, tied) -> Head
