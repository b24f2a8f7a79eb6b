"""The engine: a loaded model, its cache, and one step function.

`Engine.step(entries)` takes a batch of (request, its next tokens, wanted
places): portions of prompts beside single decoded tokens, cut anywhere.  It
runs only the tokens it is given, as one packed batch, against what earlier
steps left in the cache, and returns fp32 logits at the wanted places, in the
order of the entries and of each entry's `want`.

The reference issues a decode call and a separate prefill call per scheduler
iteration (`engine/src/runtime.rs:448-465`) and validates a packed batch before
any device write (`engine/src/gpu_model.rs:2809-2934`); here both kinds of work
are rows of one batch, and the same validation happens first.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, GroupPolicy, RELEASED
from ..config.registry import load_config
from ..models.decoder import DecoderModel
from ..weights.loader import load_weights
from .context import CacheStorage, HostStep, Scratch, StepContext, StepLayout

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
    elif name in _DTYPES:
        return _DTYPES[name]
    raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)   # places among `tokens`


class StepError(ValueError):
    pass


@dataclass
class EngineOptions:
    dtype: object = "bfloat16"
    page_tokens: int = 16                 # the reference's PAGE_TOKENS (paged.rs:51)
    n_pages: Optional[int] = None         # per cache group; default: max_requests full contexts
    max_requests: int = 16                # the reference's --max-batch default (main.rs:143)
    device: str = "cuda:0"
    graph: bool = True                    # replay decode-only steps as CUDA graphs


class Engine:
    def __init__(self, model_dir: str, options: Optional[EngineOptions] = None):
        self.options = options or EngineOptions()
        self.dtype = parse_dtype(self.options.dtype)
        if not torch.cuda.is_available():
            raise RuntimeError("crucible_b200 runs on a CUDA device (sm_100a); "
                               "torch.cuda.is_available() is False and there is no CPU path")
        self.device = torch.device(self.options.device)
        torch.cuda.set_device(self.device)
        self.config = load_config(model_dir)
        self.model = DecoderModel(self.config)
        load_weights(self.model, model_dir, self.dtype, self.device)
        self._build_storage()

    # -- storage ----------------------------------------------------------------

    def _build_storage(self) -> None:
        o = self.options
        if o.page_tokens <= 0:
            raise ValueError("page_tokens must be positive")
        ctx_pages = -(-self.config.max_context // o.page_tokens)
        n_pages = o.n_pages if o.n_pages is not None else o.max_requests * ctx_pages
        groups = self.model.cache_groups
        self.cache = CacheManager(
            [GroupPolicy(o.page_tokens, g.need.window) for g in groups],
            [n_pages] * len(groups), o.max_requests)
        self.storages = [CacheStorage(len(g.layers), n_pages, o.page_tokens, g.need.kv_heads,
                                      g.need.head_dim, self.dtype, self.device) for g in groups]
        self.table_strides = tuple(ctx_pages for _ in groups)
        self.state = None
        if self.model.state_bytes:
            self.state = torch.zeros((o.max_requests, self.model.state_bytes),
                                     dtype=torch.uint8, device=self.device)
        self.scratch = Scratch(self.device)
        self._meta_dev = None
        self._meta_host = None
        self._sampler = None
        self._graphs = {}
        self._graph_generation = 0
        self._graph_failed = False
        self._graph_error = None

    def _meta_buffers(self, n: int):
        if self._meta_dev is None or self._meta_dev.numel() < n:
            cap = max(n, 1024)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self.scratch.generation += 1
        return self._meta_host, self._meta_dev

    # -- what the scheduler needs of an executor ----------------------------------

    @property
    def vocab_size(self) -> int:
        return self.config.vocab_size

    @property
    def max_context(self) -> int:
        return self.config.max_context

    @property
    def max_device_top_k(self) -> int:
        from .. import ops
        return ops.max_device_top_k()

    def sample(self, logits: torch.Tensor, rows) -> List[int]:
        if self._sampler is None:
            from ..sampling.sampler import Sampler
            self._sampler = Sampler(self.device, self.config.vocab_size)
        return self._sampler.sample(logits, rows)

    # -- requests ---------------------------------------------------------------

    def add_request(self, request, lifetime_tokens: Optional[int] = None,
                    max_step_tokens: Optional[int] = None) -> None:
        slot = self.cache.add_request(request, lifetime_tokens, max_step_tokens)
        if self.state is not None:
            self.state[slot].zero_()      # a slot is handed out clean

    def has_request(self, request) -> bool:
        return self.cache.has(request)

    def finish(self, request) -> None:
        """Gives back everything the request holds.  Call between steps only."""
        self.cache.remove_request(request)

    def held_tokens(self, request) -> int:
        return self.cache.length(request)

    # -- the step ---------------------------------------------------------------

    def step(self, entries: Sequence[StepEntry],
             token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs one packed batch.  Returns fp32 logits [wanted, vocab] on the
        device; the tensor is scratch of the engine and is overwritten by the
        next step.  `token_source`, if given, is a device int32 tensor whose
        first rows replace the entries' token ids on the device (ids chosen by
        the previous step need not visit the host; the entries' own ids are
        then placeholders and are not validated against it)."""
        entries = list(entries)
        self._validate(entries)
        extended, added = [], []
        try:
            for e in entries:
                if not self.cache.has(e.request):
                    self.add_request(e.request)
                    added.append(e.request)
                self.cache.extend(e.request, len(e.tokens))
                extended.append(e)
        except Exception:
            # a step that cannot get its pages changes nothing
            for e in extended:
                self._shrink(e.request, len(e.tokens))
            for request in added:
                self.cache.remove_request(request)
            raise
        ctx = self._make_context(entries)
        if token_source is not None:
            ctx.token_ids.copy_(token_source[:ctx.n_tokens])
        if (self.options.graph and not self._graph_failed and ctx.host.all_single_token
                and self.model.graph_safe):
            return self._replay_or_capture(ctx)
        return self.model.forward(ctx)

    # -- CUDA graphs for decode-only steps ----------------------------------------
    #
    # A step in which every request brings one token has a launch sequence that
    # depends only on (rows, wanted rows, context bucket); the metadata it reads
    # lies at fixed addresses and is uploaded before the replay, outside the
    # graph (as `engine/src/gpu_model.rs:1348-1380`: graphs keyed by exact batch
    # size, metadata H2D before the launch).  A capture that fails is remembered
    # and the engine stays eager (`gpu_model.rs:3199-3222`).

    def _replay_or_capture(self, ctx: StepContext) -> torch.Tensor:
        from .. import ops
        if self._graph_generation != self.scratch.generation:
            self._graphs.clear()
            self._graph_generation = self.scratch.generation
        key = (ctx.n_tokens, ctx.n_logit_rows, ctx.host.context_bucket)
        hit = self._graphs.get(key)
        if hit is not None:
            graph, logits, launches = hit
            graph.replay()
            ops.LAUNCHES[0] += launches
            return logits
        logits = self.model.forward(ctx)           # eager: also sizes the scratch buffers
        if self._graph_generation != self.scratch.generation:
            self._graphs.clear()
            self._graph_generation = self.scratch.generation
        try:
            before = ops.LAUNCHES[0]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                captured = self.model.forward(ctx)
            launches = ops.LAUNCHES[0] - before
            ops.LAUNCHES[0] = before
            if self._graph_generation != self.scratch.generation:
                raise RuntimeError("scratch buffers moved during capture")
            self._graphs[key] = (graph, captured, launches)
        except Exception as e:                      # stay eager from here on
            self._graph_failed = True
            self._graph_error = repr(e)
        return logits

    def _shrink(self, request, n: int) -> None:
        r = self.cache._get(request)
        r.length -= n
        for g, pool in enumerate(self.cache.pools):
            needed = -(-r.length // pool.page_tokens)
            while len(r.tables[g]) > needed:
                pool.release(r.tables[g].pop())

    def _validate(self, entries: List[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        new_requests = 0
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            held = self.cache.length(e.request) if self.cache.has(e.request) else 0
            if not self.cache.has(e.request):
                new_requests += 1
            if held + n > self.config.max_context:
                raise StepError(f"request {e.request!r} would hold {held + n} tokens; the "
                                f"model's context is {self.config.max_context}")
            for tok in e.tokens:
                if not 0 <= int(tok) < self.config.vocab_size:
                    raise StepError(f"request {e.request!r}: token {tok} is outside the "
                                    f"vocabulary of {self.config.vocab_size}")
            last = -1
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its "
                                    f"{n} tokens")
                if int(w) <= last:
                    raise StepError(f"request {e.request!r}: wanted places must ascend")
                last = int(w)
        if new_requests > self.cache.slots.free_slots:
            raise StepError(f"{new_requests} new requests but only "
                            f"{self.cache.slots.free_slots} of {self.options.max_requests} "
                            f"request slots are free")

    def _make_context(self, entries: List[StepEntry]) -> StepContext:
        n_tokens = sum(len(e.tokens) for e in entries)
        n_want = sum(len(e.want) for e in entries)
        layout = StepLayout(n_tokens, len(entries), n_want, self.table_strides)
        off = layout.offsets()
        total = off["_total"][1]
        host_t, dev_t = self._meta_buffers(total)
        host = host_t.numpy()

        def piece(name):
            a, n = off[name]
            return host[a:a + n]

        token_ids, positions = piece("token_ids"), piece("positions")
        row_request, logit_rows = piece("row_request"), piece("logit_rows")
        row_start, ctx_len = piece("req_row_start"), piece("req_context_len")
        first_pos, state_slot = piece("req_first_pos"), piece("req_state_slot")
        hs = HostStep([], [], [], [], [])
        row = 0
        w_at = 0
        for r, e in enumerate(entries):
            n = len(e.tokens)
            held_after = self.cache.length(e.request)
            start = held_after - n
            token_ids[row:row + n] = np.asarray(e.tokens, dtype=np.int32)
            positions[row:row + n] = np.arange(start, held_after, dtype=np.int32)
            row_request[row:row + n] = r
            for w in e.want:
                logit_rows[w_at] = row + int(w)
                w_at += 1
            row_start[r] = row
            ctx_len[r] = held_after
            first_pos[r] = start
            slot = self.cache.state_slot(e.request)
            state_slot[r] = slot
            hs.request_ids.append(e.request)
            hs.new_tokens.append(n)
            hs.first_pos.append(start)
            hs.context_len.append(held_after)
            hs.state_slots.append(slot)
            for g, stride in enumerate(self.table_strides):
                table = self.cache.block_table(e.request, g)
                a, _ = off[f"table{g}"]
                dst = host[a + r * stride:a + (r + 1) * stride]
                dst[:len(table)] = table
                dst[len(table):] = 0
                n_pages = self.cache.pools[g].n_pages
                for p in table:
                    if p != RELEASED and not 0 <= p < n_pages:
                        raise StepError(f"page {p} of request {e.request!r} is out of range")
            row += n
        row_start[len(entries)] = row
        dev_t[:total].copy_(host_t[:total], non_blocking=True)
        return StepContext(layout=layout, meta=dev_t, caches=self.storages, state=self.state,
                           scratch=self.scratch, dtype=self.dtype, host=hs)
