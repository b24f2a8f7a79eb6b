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

import ctypes
from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, GroupPolicy
from ..cache import pages as cache_codes
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


class _Packer:
    """The native step packer (`csrc/host_step.cpp`) with its constant arguments."""

    def __init__(self, table_strides):
        from ..ops import build
        lib = build.load("host_step")
        self.fn = lib.cb_host_pack_step
        self.fn.restype = ctypes.c_int
        self.fn.argtypes = ([ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6
                            + [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                               ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_char_p,
                               ctypes.c_int])
        self._strides = (ctypes.c_int32 * max(1, len(table_strides)))(*table_strides)
        self.strides = ctypes.cast(self._strides, ctypes.c_void_p)
        self.err = ctypes.create_string_buffer(256)


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)   # places among `tokens`


class _Choice:
    """The greedy choice of a choosing step: the state slots of its rows, the device buffers
    the argmax writes (ids with the status word behind them, the slots as the kernel reads
    them) and, for a captured step, the event behind the last copy of the ids to the host."""

    def __init__(self, slots_key):
        self.slots_key = slots_key
        self.ids = None
        self.slots = None
        self.copied = None
        self.keeper = None      # the captured step's own choice, if this one borrowed its buffers


class StepError(ValueError):
    pass


# As the only token of an entry: "the token the engine last chose for this request",
# which it kept on the device (see `Engine.sample`); the host need not know it yet.
DEVICE_TOKEN = -1


@dataclass
class EngineOptions:
    dtype: object = "bfloat16"
    page_tokens: int = 16                 # the reference's PAGE_TOKENS (paged.rs:51)
    n_pages: Optional[int] = None         # per cache group; default: max_requests full contexts
    max_requests: int = 16                # the reference's --max-batch default (main.rs:143)
    device: str = "cuda:0"
    graph: bool = True                    # replay decode-only steps as CUDA graphs
    profile: bool = False                 # CUDA events around every part's forward; steps run eagerly


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
        self.profiler = None
        if self.options.profile:
            from .profile import StageProfiler, attach
            self.profiler = StageProfiler()
            attach(self.model, self.profiler)
        self._build_storage()

    # -- storage ----------------------------------------------------------------

    def _build_storage(self) -> None:
        o = self.options
        if o.page_tokens <= 0:
            raise ValueError("page_tokens must be positive")
        ctx_pages = -(-self.config.max_context // o.page_tokens)
        n_pages = o.n_pages if o.n_pages is not None else o.max_requests * ctx_pages
        groups = self.model.cache_groups
        # One page more than the pool hands out: the null page, never written, all zeros.
        # A table entry whose page the window has passed and given back names it, so a
        # kernel that loads whole tiles of keys reads zeros there (every such key is masked)
        # and never another request's data.
        self.storages = [CacheStorage(len(g.layers), n_pages + 1, o.page_tokens, g.need.kv_heads,
                                      g.need.head_dim, self.dtype, self.device) for g in groups]
        self.null_page = n_pages
        self.table_strides = tuple(ctx_pages for _ in groups)
        # The manager keeps every live request's table in the form that goes to the device
        # (a row of the table stride at a fixed address) and its own ledger of which request
        # names which page: a step whose growth would let two requests name one page is
        # refused before anything is written (`engine/src/gpu_model.rs:2809-2934` refuses
        # such a batch).
        self.cache = CacheManager(
            [GroupPolicy(o.page_tokens, g.need.window) for g in groups],
            [n_pages] * len(groups), o.max_requests, table_strides=self.table_strides,
            null_pages=[self.null_page] * len(groups))
        self._has_device_token = set()      # state slots whose latest token is on the device
        self.state = None
        if self.model.state_bytes:
            self.state = torch.zeros((o.max_requests, self.model.state_bytes),
                                     dtype=torch.uint8, device=self.device)
        self.scratch = Scratch(self.device)
        self.device_tokens = torch.zeros(o.max_requests, dtype=torch.int32, device=self.device)
        self._meta_dev = None
        self._meta_ring = []
        self._sampler = None
        self._graphs = {}
        self._graph_generation = 0
        self._graph_failed = False
        self._graph_error = None
        self._graph_replays = 0          # steps run by replaying a captured graph ...
        self._prompt_graph_replays = 0   # ... of which steps that held a prompt portion
        from ..ops import tensor_core
        self._failures_seen = tensor_core.FAILURES[0]
        self._shapes_seen = {}
        self._packer = _Packer(self.table_strides)

    META_RING = 4

    def _meta_buffers(self, n: int):
        """The device metadata buffer for this step (one of two, at fixed addresses, taken
        in turn) and a pinned host buffer to fill.  The upload is asynchronous and runs on a
        stream of its own, so that a step's metadata crosses while the step before it still
        runs (between two replayed graphs the copy and the gaps around it were 12 us of a
        0.32 ms step).  The host may run ahead of the device by several steps: the pinned
        buffers form a ring, and one is reused only after the copy that last read it has
        finished; a device buffer is written only after the step that last read it has run."""
        if self._meta_dev is None or self._meta_dev[0].numel() < n:
            cap = max(n, 1024)
            torch.cuda.synchronize(self.device)
            self._meta_dev = [torch.empty(cap, dtype=torch.int32, device=self.device) for _ in range(2)]
            self._meta_ready = [torch.cuda.Event() for _ in range(2)]   # the step's metadata has landed
            self._meta_free = [torch.cuda.Event() for _ in range(2)]    # the step that read it has run
            self._meta_dev_at = 0
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._meta_ring = [(torch.empty(cap, dtype=torch.int32, pin_memory=True),
                                torch.cuda.Event()) for _ in range(self.META_RING)]
            self._meta_used = [False] * self.META_RING
            self._meta_at = 0
            self.scratch.generation += 1
        self._meta_at = (self._meta_at + 1) % self.META_RING
        self._meta_dev_at ^= 1
        host, event = self._meta_ring[self._meta_at]
        if self._meta_used[self._meta_at]:
            event.synchronize()
        return host, self._meta_dev[self._meta_dev_at]

    def _upload_meta(self, host_t: torch.Tensor, total: int) -> None:
        d, copies = self._meta_dev_at, self._copy_stream
        copies.wait_event(self._meta_free[d])
        with torch.cuda.stream(copies):
            self._meta_dev[d][:total].copy_(host_t[:total], non_blocking=True)
            self._meta_ring[self._meta_at][1].record(copies)
            self._meta_ready[d].record(copies)
        self._meta_used[self._meta_at] = True
        torch.cuda.current_stream(self.device).wait_event(self._meta_ready[d])

    def _meta_read(self) -> None:
        """Called when a step's launches are in the stream: its metadata buffer may be
        written again once they have run."""
        self._meta_free[self._meta_dev_at].record(torch.cuda.current_stream(self.device))

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

    def _get_sampler(self):
        if self._sampler is None:
            from ..sampling.sampler import Sampler
            self._sampler = Sampler(self.device, self.config.vocab_size)
        return self._sampler

    def sample(self, logits: torch.Tensor, rows) -> List[int]:
        """Chooses a token for every row of `logits`; returns the ids."""
        return self._get_sampler().sample(logits, rows)

    def sample_deferred(self, logits: torch.Tensor, rows, requests):
        """Chooses a token for every row and keeps it on the device as the latest
        token of `requests[i]` (an entry with tokens [DEVICE_TOKEN] runs it).  The
        ids travel to the host asynchronously; the returned object's `get()` waits
        for them."""
        slots = [self.cache.state_slot(r) for r in requests]
        self._has_device_token.update(slots)
        return self._get_sampler().sample(logits, rows, slots=slots,
                                          scatter_out=self.device_tokens, defer=True)

    # -- requests ---------------------------------------------------------------

    def add_request(self, request, lifetime_tokens: Optional[int] = None,
                    max_step_tokens: Optional[int] = None) -> None:
        slot = self.cache.add_request(request, lifetime_tokens, max_step_tokens)
        self._has_device_token.discard(slot)   # the slot's last owner's token is not this one's
        if self.state is not None:
            self.state[slot].zero_()      # a slot is handed out clean

    def has_request(self, request) -> bool:
        return self.cache.has(request)

    def finish(self, request) -> None:
        """Gives back everything the request holds.  Call between steps only."""
        self._forget(request)
        self.cache.remove_request(request)

    def _forget(self, request) -> None:
        """Drops what the engine itself remembers of a request that is about to go."""
        self._has_device_token.discard(self.cache.state_slot(request))

    def held_tokens(self, request) -> int:
        return self.cache.length(request)

    # -- the step ---------------------------------------------------------------

    def step_choosing(self, entries: Sequence[StepEntry]):
        """A step whose every entry wants the logits of its last token and chooses its next
        token greedily, the choice being part of the step: for a step that replays a captured
        graph the argmax is a kernel of that graph, not a launch behind it.  The chosen
        tokens stay on the device as the requests' latest (as `sample_deferred` leaves them).
        Returns (logits, ids on their way to the host)."""
        entries = list(entries)
        for e in entries:
            if list(e.want) != [len(e.tokens) - 1]:
                raise StepError("step_choosing: every entry wants the logits of its last token, and no others")
        return self.step(entries, _choose=True)

    def step(self, entries: Sequence[StepEntry],
             token_source: Optional[torch.Tensor] = None, _choose: bool = False) -> torch.Tensor:
        """Runs one packed batch.  Returns fp32 logits [wanted, vocab] on the
        device; the tensor is scratch of the engine and is overwritten by the
        next step.  `token_source`, if given, is a device int32 tensor whose
        first rows replace the entries' token ids on the device (ids chosen by
        the previous step need not visit the host; the entries' own ids are
        then placeholders and are not validated against it)."""
        entries = list(entries)
        self._validate(entries)
        cache = self.cache
        n_req = len(entries)
        added, grown, ints = [], False, None
        try:
            for e in entries:
                if not cache.has(e.request):
                    self.add_request(e.request)
                    added.append(e.request)
            counts = [len(e.tokens) for e in entries]
            # rows: token counts, first positions (filled by the manager), slots, wanted counts
            ints = np.array([counts, counts, [cache.state_slot(e.request) for e in entries],
                             [len(e.want) for e in entries]], dtype=np.int32)
            rows = (ctypes.c_void_p * max(1, len(self.table_strides) * n_req))()
            # every request's pages for this step, or nobody's; the tables that will go to
            # the device come back as the addresses of the manager's rows
            code = cache.step_raw(n_req, ints[2].ctypes.data, ints[0].ctypes.data,
                                  self.config.max_context, ints[1].ctypes.data, rows)
            if code:
                who = entries[cache.failed_entry()].request
                if code in (cache_codes.TOO_LONG, cache_codes.ALIASED):
                    raise StepError(f"request {who!r}: {cache._message()}")
                cache.raise_for(code, who)
            grown = True
            ctx = self._make_context(entries, ints, rows)
        except Exception:
            # a step that cannot get its pages, or whose tables or tokens are not sound,
            # changes nothing
            if grown:
                cache.unstep_raw(n_req, ints[2].ctypes.data, ints[0].ctypes.data)
            for request in added:
                self._forget(request)
                cache.remove_request(request)
            raise
        choice = None
        if _choose:
            slots = ints[2].tolist()
            self._has_device_token.update(slots)
            choice = _Choice(tuple(slots))
        try:
            if token_source is not None:
                ctx.token_ids.copy_(token_source[:ctx.n_tokens])
            logits = None
            if self.profiler is not None:
                self.profiler.steps += 1
            elif self.options.graph and not self._graph_failed:
                if ctx.host.all_single_token:
                    if self.model.graph_safe:
                        logits = self._replay_or_capture(ctx, at_once=True, choice=choice)
                elif self.model.graph_safe_prompt_steps:
                    logits = self._replay_or_capture(ctx, at_once=False, choice=choice)
            if logits is None:
                logits = self.model.forward(ctx)
                if choice is not None:
                    self._choose(logits, choice)
        finally:
            self._meta_read()
        if choice is None:
            return logits
        return logits, self._get_sampler().collect(choice.ids, len(choice.slots_key), choice)

    def _choose(self, logits: torch.Tensor, choice: "_Choice") -> None:
        """The argmax of a choosing step, into the choice's own buffers (a captured step keeps
        them: they are what its kernels write)."""
        from .. import ops
        from ..ops import tensor_core
        n = len(choice.slots_key)
        if choice.ids is None:
            choice.ids = torch.zeros(n + 1, dtype=torch.int32, device=self.device)
            choice.slots = torch.tensor(choice.slots_key, dtype=torch.int32, device=self.device)
        # the kernel that writes the ids also leaves the status word right behind them
        status = (tensor_core.status_word(self.device), choice.ids[n:n + 1])
        ops.argmax_rows(logits, choice.ids[:n], choice.slots, self.device_tokens, status=status)

    # -- CUDA graphs ----------------------------------------------------------------
    #
    # The launch sequence of a step depends only on its shape: (rows, requests,
    # wanted rows, most new tokens of a request, context bucket); everything else
    # the kernels read from metadata at fixed addresses, uploaded before the replay
    # and outside the graph (as `engine/src/gpu_model.rs:1348-1380`: decode graphs
    # keyed by exact batch size, metadata H2D before the launch; and `:3193-3229`:
    # prefill graphs keyed by length, at most 64 of them).  A decode-only shape is
    # captured the first time it is seen, any other shape the second time.  A
    # capture that fails is remembered and the engine stays eager
    # (`gpu_model.rs:3199-3222`).

    MAX_GRAPHS = 128         # two to a shape: one for each metadata buffer

    def _replay_or_capture(self, ctx: StepContext, at_once: bool, choice=None) -> torch.Tensor:
        from .. import ops
        from ..ops import tensor_core
        if self._failures_seen != tensor_core.FAILURES[0]:
            # a kernel gave up since the last step: what was captured is kept no longer
            self._failures_seen = tensor_core.FAILURES[0]
            self._graphs.clear()
            self._shapes_seen.clear()
        if self._graph_generation != self.scratch.generation:
            self._graphs.clear()
            self._graph_generation = self.scratch.generation
        host = ctx.host
        shape = (ctx.n_tokens, ctx.n_requests, ctx.n_logit_rows) + host.shape_key()
        # a graph's kernels read one of the two metadata buffers; a choosing step's graph also
        # holds its argmax
        key = shape + (self._meta_dev_at, choice is not None)
        hit = self._graphs.get(key)
        if hit is not None:
            graph, logits, launches, kept = hit
            if choice is not None:
                # the graph writes the buffers of the choice it was captured with
                if kept.slots_key != choice.slots_key:
                    kept.slots.copy_(torch.tensor(choice.slots_key, dtype=torch.int32))
                    kept.slots_key = choice.slots_key
                if kept.copied is not None:
                    # its ids of last time have to be on their way out before they are overwritten
                    torch.cuda.current_stream(self.device).wait_event(kept.copied)
                choice.ids, choice.slots, choice.keeper = kept.ids, kept.slots, kept
            graph.replay()
            ops.LAUNCHES[0] += launches
            self._graph_replays += 1
            self._prompt_graph_replays += 0 if at_once else 1
            return logits
        logits = self.model.forward(ctx)           # eager: also sizes the scratch buffers
        if choice is not None:
            self._choose(logits, choice)
        if self._graph_generation != self.scratch.generation:
            self._graphs.clear()
            self._graph_generation = self.scratch.generation
        if not at_once:
            seen = self._shapes_seen.get(shape, 0) + 1
            self._shapes_seen[shape] = seen
            if seen < 2:
                return logits
            if len(self._shapes_seen) > 4096:
                self._shapes_seen.clear()
        try:
            before = ops.LAUNCHES[0]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                captured = self.model.forward(ctx)
                if choice is not None:
                    self._choose(captured, choice)
            launches = ops.LAUNCHES[0] - before
            ops.LAUNCHES[0] = before
            if self._graph_generation != self.scratch.generation:
                raise RuntimeError("scratch buffers moved during capture")
            while len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = (graph, captured, launches, choice)
        except Exception as e:                      # stay eager from here on
            self._graph_failed = True
            self._graph_error = repr(e)
        return logits

    def _validate(self, entries: List[StepEntry]) -> None:
        """What can be said of a step before the cache is asked.  The rest is checked
        natively as the step is built, and a failure there is rolled back like a failed
        allocation: a context too long by the cache manager as it grows the request, token
        ids and wanted places by the packer as it writes them."""
        if not entries:
            raise StepError("a step needs at least one entry")
        cache = self.cache
        seen = set()
        new_requests = 0
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            known = cache.has(e.request)
            if n == 1 and e.tokens[0] == DEVICE_TOKEN:
                if not known or cache.state_slot(e.request) not in self._has_device_token:
                    raise StepError(f"request {e.request!r} has no token on the device yet")
            if not known:
                new_requests += 1
                if n > self.config.max_context:
                    raise StepError(f"request {e.request!r} would hold {n} tokens; the "
                                    f"model's context is {self.config.max_context}")
        if new_requests and new_requests > cache.slots.free_slots:
            raise StepError(f"{new_requests} new requests but only "
                            f"{cache.slots.free_slots} of {self.options.max_requests} "
                            f"request slots are free")

    def check_tables(self) -> None:
        """The whole check, over every live request and not only the pages new to a step:
        no page of a cache group is named by two requests, or twice by one.  Growth checks
        the pages it adds; this is for tests and for a host that suspects its allocator."""
        from ..cache import CacheError
        try:
            self.cache.check_tables()
        except CacheError as e:
            raise StepError(str(e)) from None

    def _make_context(self, entries: List[StepEntry], ints: np.ndarray, rows) -> StepContext:
        """Packs the step's metadata into a pinned block (the native packer,
        `csrc/host_step.cpp`, which also checks every token id and wanted place) and
        sends it to the device.  `ints`: int32 rows of token counts, first positions, state
        slots and wanted counts, one column per entry; `rows`: addresses of the requests'
        table rows, group after group."""
        n_req = len(entries)
        counts, starts, slots, want_counts = ints.tolist()
        n_tokens, n_want = sum(counts), sum(want_counts)
        layout = StepLayout(n_tokens, n_req, n_want, self.table_strides)
        total = layout.offsets()["_total"][1]
        host_t, dev_t = self._meta_buffers(total)
        held_after = [s + n for s, n in zip(starts, counts)]
        if n_tokens == n_req:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=n_req)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if n_want == n_req and all(c == 1 for c in want_counts):
            wants = np.fromiter((e.want[0] for e in entries), dtype=np.int32, count=n_req)
        else:
            wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=n_want)
        pack = self._packer
        n_groups = len(self.table_strides)
        bad = ctypes.c_int32(-1)
        code = pack.fn(host_t.data_ptr(), n_req, ints[0].ctypes.data, ints[1].ctypes.data,
                       ints[2].ctypes.data, tokens.ctypes.data, ints[3].ctypes.data,
                       wants.ctypes.data, n_groups, pack.strides, rows, self.config.vocab_size,
                       self.config.max_context, DEVICE_TOKEN, ctypes.byref(bad), pack.err, 256)
        if code != 0:
            who = entries[bad.value].request if 0 <= bad.value < n_req else None
            raise StepError(f"request {who!r}: {pack.err.value.decode()}")
        hs = HostStep([e.request for e in entries], counts, starts, held_after, slots)
        self._upload_meta(host_t, total)
        return StepContext(layout=layout, meta=dev_t, caches=self.storages, state=self.state,
                           scratch=self.scratch, dtype=self.dtype, host=hs,
                           device_tokens=self.device_tokens)
