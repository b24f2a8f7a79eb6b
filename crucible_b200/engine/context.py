"""What one step looks like to the model: the packed batch and its storage.

`StepLayout` fixes where each piece of a step's integer metadata lies inside
one int32 buffer, as a function of the step's row, request and wanted-row
counts only; the host fills a pinned copy and uploads it with a single copy.
`StepContext` is what parts see: device views of that metadata, the cache
storage of each group, per-request state, and named scratch buffers.

The packed-batch idea follows the reference's packed prefill
(`engine/src/gpu_model.rs:256-272`, `:2872-2896`: owners, positions, segments,
final rows) extended so that a decoded token is simply a portion of length one.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import cached_property, lru_cache
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class StepLayout:
    n_tokens: int
    n_requests: int
    n_logit_rows: int
    table_strides: Tuple[int, ...]

    def offsets(self) -> Dict[str, Tuple[int, int]]:
        """name -> (offset, length) in ints; the native packer (`csrc/host_step.cpp`) lays
        a step out by the same rule."""
        return _offsets(self)


@lru_cache(maxsize=256)
def _offsets(layout: "StepLayout") -> Dict[str, Tuple[int, int]]:
    t, r, f = layout.n_tokens, layout.n_requests, layout.n_logit_rows
    out, at = {}, 0
    for name, n in (("token_ids", t), ("positions", t), ("row_request", t),
                    ("logit_rows", f), ("req_row_start", r + 1), ("req_context_len", r),
                    ("req_first_pos", r), ("req_state_slot", r)):
        out[name] = (at, n)
        at += (n + 3) // 4 * 4            # keep every piece 16-byte aligned
    for g, stride in enumerate(layout.table_strides):
        out[f"table{g}"] = (at, r * stride)
        at += (r * stride + 3) // 4 * 4
    out["_total"] = (0, at)
    return out


class CacheStorage:
    """Device pages of one cache group: [slot, K|V, page, kv_head, token, feature].
    Inside a page each KV head's tokens are contiguous (page_tokens * head_dim
    elements in a row), so a head's keys are read in long runs."""

    def __init__(self, n_slots: int, n_pages: int, page_tokens: int, kv_heads: int,
                 head_dim: int, dtype: torch.dtype, device):
        self.page_tokens = page_tokens
        self.n_pages = n_pages
        self.kv_heads = kv_heads
        self.head_dim = head_dim
        self.kv = torch.zeros((n_slots, 2, n_pages, kv_heads, page_tokens, head_dim),
                              dtype=dtype, device=device)

    def keys(self, slot: int) -> torch.Tensor:
        return self.kv[slot, 0]

    def values(self, slot: int) -> torch.Tensor:
        return self.kv[slot, 1]


class Scratch:
    """Named device buffers that persist between steps (stable addresses while
    their size suffices), so a step allocates nothing once warmed up."""

    def __init__(self, device):
        self.device = device
        self._flat: Dict[str, torch.Tensor] = {}
        self.generation = 0          # bumped whenever a buffer moves

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        key = f"{name}:{dtype}"
        flat = self._flat.get(key)
        if flat is None or flat.numel() < numel:
            flat = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
            self.generation += 1
        return flat[:numel].view(*shape)

    def reserve(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> None:
        self.get(name, shape, dtype)


class StepContext:
    """Everything a part may know about the step being run."""

    def __init__(self, *, layout: StepLayout, meta: torch.Tensor, caches: List[CacheStorage],
                 state: Optional[torch.Tensor], scratch: Scratch, dtype: torch.dtype,
                 host: "HostStep", device_tokens: Optional[torch.Tensor] = None):
        self.layout = layout
        self.dtype = dtype
        self.n_tokens = layout.n_tokens
        self.n_requests = layout.n_requests
        self.n_logit_rows = layout.n_logit_rows
        self._caches = caches
        self._state = state
        self._scratch = scratch
        self.host = host
        self.device_tokens = device_tokens     # int32 per state slot: the token last chosen
        off = layout.offsets()

        def view(name):
            a, n = off[name]
            return meta[a:a + n]

        self.token_ids = view("token_ids")
        self.positions = view("positions")
        self.row_request = view("row_request")
        self.logit_rows = view("logit_rows")
        self.req_row_start = view("req_row_start")
        self.req_context_len = view("req_context_len")
        self.req_first_pos = view("req_first_pos")
        self.req_state_slot = view("req_state_slot")
        self._tables = [view(f"table{g}").view(layout.n_requests, s)
                        for g, s in enumerate(layout.table_strides)]

    def cache(self, group: int) -> CacheStorage:
        return self._caches[group]

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    def state(self, binding) -> Optional[torch.Tensor]:
        """The mixer's bytes inside every request's state slot: uint8
        [n_slots, state_bytes]; index it with `req_state_slot`."""
        if self._state is None or binding.state_bytes == 0:
            return None
        return self._state[:, binding.state_offset:binding.state_offset + binding.state_bytes]

    def scratch(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        return self._scratch.get(name, shape, dtype)

    # -- a norm announced to the product that writes its rows last ------------
    # An arrangement that knows which norm reads the residual rows next, through a consumer
    # that can take rows not yet normalised, announces it before it runs the part in between.
    # That part's last product into the rows (`ops.linear(..., accumulate=True, closes=ctx)`)
    # may then leave the norm's input beside its sums and offer it; the norm takes the offer
    # instead of running a kernel.  Nothing has to happen: an announcement that no product
    # honours, or an offer that no norm takes, costs nothing and changes no result.
    norm_after_layer = None      # set by the model before each layer: (norm, consumer) of the
                                 # layer that runs next, or None
    _announced = None            # (norm, address and shape of the rows it will read)
    _offer = None                # (norm, address and shape of the rows, scaled, sumsq, parts)

    def announce_norm(self, norm, rows: Optional[torch.Tensor]) -> None:
        self._announced = (norm, rows.data_ptr(), tuple(rows.shape)) if norm is not None else None
        self._offer = None

    def norm_ahead(self, rows: torch.Tensor):
        a = self._announced
        if a is None or a[1] != rows.data_ptr() or a[2] != tuple(rows.shape):
            return None
        return a[0]

    def offer_prenormed(self, rows: torch.Tensor, norm, scaled, sumsq, parts: int) -> None:
        self._offer = (norm, rows.data_ptr(), tuple(rows.shape), scaled, sumsq, parts)
        self._announced = None

    def take_prenormed(self, rows: torch.Tensor, norm):
        o, self._offer = self._offer, None
        self._announced = None
        if o is None or o[0] is not norm or o[1] != rows.data_ptr() or o[2] != tuple(rows.shape):
            return None
        return o[3], o[4], o[5]


@dataclass
class HostStep:
    """Host-side copy of the step's shape, for parts that pick a launch shape."""
    request_ids: list
    new_tokens: List[int]            # per request: tokens run in this step
    first_pos: List[int]             # per request: position of its first new token
    context_len: List[int]           # per request: tokens held after this step
    state_slots: List[int]

    @cached_property
    def all_single_token(self) -> bool:
        return all(n == 1 for n in self.new_tokens)

    @cached_property
    def max_context_len(self) -> int:
        return max(self.context_len) if self.context_len else 0

    @cached_property
    def max_new_tokens(self) -> int:
        return max(self.new_tokens) if self.new_tokens else 0

    @staticmethod
    def _bucket(longest: int) -> int:
        return 256 * max(1, -(-longest // 256))

    @cached_property
    def context_bucket(self) -> int:
        """The longest context of the step rounded up to a multiple of 256.  Launch
        shapes that depend on context length use this, so that a captured step can
        be replayed for any context inside the bucket."""
        return self._bucket(self.max_context_len)

    @cached_property
    def lead_single(self) -> int:
        """How many requests at the head of the step bring exactly one token (the
        scheduler puts decoding requests first)."""
        n = 0
        for k in self.new_tokens:
            if k != 1:
                break
            n += 1
        return n

    @cached_property
    def lead_context_bucket(self) -> int:
        """`context_bucket` over the leading single-token requests alone (0: none)."""
        n = self.lead_single
        return self._bucket(max(self.context_len[:n])) if n else 0

    SMALL_STEP_TOKENS = 16

    def shape_key(self) -> tuple:
        """What, beside the counts of rows, requests and wanted rows, a kernel's launch
        shape may depend on: the most new tokens of a request, the number of leading
        single-token requests, and the context buckets of the requests that may run
        split over their keys (all of them when every request brings few tokens; the
        leading single-token ones otherwise).  Steps with equal keys launch the same
        kernels with the same grids."""
        small = self.max_new_tokens <= self.SMALL_STEP_TOKENS
        return (self.max_new_tokens, self.lead_single,
                self.context_bucket if small else 0, self.lead_context_bucket)
