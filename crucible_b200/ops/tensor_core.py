"""The bfloat16 tensor-core kernels.  Each function returns True if it ran, or
False if the sizes are outside what the kernel takes, in which case the caller
runs the plain CUDA-core kernel instead.  The rule is stated here and depends
on the shapes and strides alone, never on the batch:

matrix products (tcgen05 + TMA): K, the row strides of both operands and the
row stride of a bfloat16 output must be multiples of 8 elements (TMA needs
16-byte row pitches), and the operand bases 16-byte aligned.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import build

build.register_module("gemm_tcgen05", ["common.cuh", "tc_common.cuh"])
build.register_module("attention_mma", ["common.cuh"])
build.register_module("gemm_skinny_tcgen05", ["common.cuh", "tc_common.cuh"])
build.register_module("attention_tcgen05", ["common.cuh", "tc_common.cuh"])
build.register_module("attention_decode_tcgen05", ["common.cuh", "tc_common.cuh"])

# Portions of prompts with head size 64 run on the tcgen05 attention kernel; False sends
# them to the mma.sync kernel instead (the tests compare the two).
USE_TCGEN05_ATTENTION = True
USE_TCGEN05_DECODE = True

_c_int, _c_void_p = ctypes.c_int, ctypes.c_void_p
STORE_BF16, STORE_F32, ACCUM_F32, SWIGLU_BF16, ROPE_APPEND = 0, 1, 2, 3, 4
_UNSUPPORTED = 100001

_status = {}
FAILURES = [0]       # kernels that gave up so far; engines drop their captured steps when it moves


class KernelGaveUp(RuntimeError):
    """A tensor-core kernel ran out one of its bounded waits: the results of the step
    it belonged to are not valid."""


def status_word(device) -> torch.Tensor:
    """A device int the kernels write if one of their bounded waits runs out."""
    key = torch.device(device).index or 0
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def raise_if_gave_up(device, code: int) -> None:
    """`code` is a value of the status word that reached the host (read here, or relayed
    behind a step's chosen ids).  Non-zero: puts the device-side state back in order (the
    word to zero; the arrival counters of the split kernels, which a block that gave up
    leaves counted short) and raises."""
    if not code:
        return
    key = torch.device(device).index or 0
    torch.cuda.synchronize(device)
    t = _status.get(key)
    if t is not None:
        t.zero_()
    for (dev, name), buf in _buffers.items():
        if dev == key and name.endswith(".counters"):
            buf.zero_()
    FAILURES[0] += 1
    what = {1: "a TMA producer", 2: "an MMA issuer", 3: "an epilogue",
            4: "a wait made to run out on purpose"}.get(code, "a role")
    raise KernelGaveUp(f"a tensor-core kernel gave up: {what} waited past its limit "
                       f"(status {code}); the step's results are not valid")


def check_status(device) -> None:
    """Raises if a tensor-core kernel gave up a wait since the last check.
    Synchronises; call it where the host waits anyway."""
    key = torch.device(device).index or 0
    t = _status.get(key)
    if t is None:
        return
    raise_if_gave_up(device, int(t.item()))


def _count(n: int) -> None:
    from . import LAUNCHES
    LAUNCHES[0] += n


def _stream():
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


TILE_WIDTHS = (64, 96, 128, 160, 192, 256)
N_SMS = 148


def _tile_of(tile):
    """`tile` as callers may give it: a width, (width, blocks per SM), or
    (width, blocks per SM, shares of K)."""
    return (tile, 1) if isinstance(tile, int) else tuple(tile)


# Shares of K, measured on B200 at 33 to 512 rows: a block's chain costs about 0.32 us per
# block of 64 elements of K (0.43 us for tiles wider than 128 columns: the ring of stages
# in flight over the latency of a load, not the tile's bytes, sets it), a cluster costs
# about 2 us more than a lone block, and the first block of a cluster takes about 0.5 us
# to pull 32 KB of another block's sums.  Clusters of 3 and 4 need room to be placed inside
# one GPC, so they may not fill the SMs to the last one.
K_SPLIT_STEP_US = (0.32, 0.43)
K_SPLIT_CLUSTER_US = 2.0
K_SPLIT_PULL_US = 0.5
K_SPLIT_BLOCK_LIMIT = {2: 148, 3: 120, 4: 128}
K_SPLIT_MIN_GAIN_US = 1.0


def k_splits(m: int, n_cols: int, k: int, bn: int) -> int:
    """Blocks that share one tile's K as a cluster (1: none).  A step of 33 to a few
    hundred rows has few tiles, each a chain of K / 64 loads and products on one SM while
    most SMs idle; shares of K spread the chain over the idle SMs."""
    tiles = -(-m // 128) * -(-n_cols // bn)
    k_blocks = -(-k // 64)
    step = K_SPLIT_STEP_US[1 if bn > 128 else 0]
    best, best_cost = 1, k_blocks * step - K_SPLIT_MIN_GAIN_US
    for s, limit in K_SPLIT_BLOCK_LIMIT.items():
        per = -(-k_blocks // s)
        if tiles * s > limit or (s - 1) * per >= k_blocks:
            continue
        cost = per * step + K_SPLIT_CLUSTER_US + K_SPLIT_PULL_US * (s - 1) * bn / 64
        if cost < best_cost:
            best, best_cost = s, cost
    return best


def _tile_width(m: int, n_cols: int, epi: int = 1, multiple_of: int = 1):
    """Tile width in output columns: the one that needs the least time if every
    block costs (width + a fixed part) and blocks run in waves over the SMs.  A
    wide tile reuses the A tile more; a narrow one fills the last wave better.
    Widths whose output cannot leave through shared memory and TMA (bfloat16 rows
    that are no multiple of 128 bytes per tile) pay for their strided stores."""
    m_tiles = -(-m // 128)
    best, best_cost = 64, None
    for bn in TILE_WIDTHS:
        if bn % multiple_of:
            continue
        blocks = m_tiles * -(-n_cols // bn)
        direct = (epi == STORE_BF16 and bn % 64) or (epi == SWIGLU_BF16 and bn % 128)
        cost = -(-blocks // N_SMS) * (bn + 48 + (40 if direct else 0))
        if best_cost is None or cost < best_cost or (cost == best_cost and bn > best):
            best, best_cost = bn, cost
    return best, 1


TALL_MIN_ROWS = 1024        # two accumulators per block (256 x 256 of output) ...
TALL_MIN_K = 512            # ... pay where many rows meet enough 256 x 256 tiles to fill the SMs: at
TALL_MIN_FILL = 0.8         # long K they halve the operand bytes per flop, at short K the blocks' starts and ends


def _tall_tiles(m: int, n_cols: int, k: int) -> bool:
    """Whether a product should run as 256 x 256 tiles (two accumulators per block).  At the
    Llama-3-8B layer sizes 148 blocks of 128 x 256 ask the L2 for 384 rows of operands per
    tile and run at half the tensor cores' rate; 256 x 256 needs 512 rows for twice the output."""
    if m < TALL_MIN_ROWS or k < TALL_MIN_K:
        return False
    blocks = -(-m // 256) * -(-n_cols // 256)
    waves = -(-blocks // N_SMS)
    return blocks / (waves * N_SMS) >= TALL_MIN_FILL


NORM_AHEAD = True    # the accumulate products may leave the next norm's input (tests switch it off)
NORM_AHEAD_MAX_TILE = 128   # widest tile whose epilogue holds a row's sums in registers


class _NormArgs(ctypes.Structure):
    """`NormArgs` of csrc/gemm_tcgen05.cu."""
    _fields_ = [("gain", ctypes.c_void_p), ("scaled", ctypes.c_void_p), ("sumsq_out", ctypes.c_void_p),
                ("ld_scaled", ctypes.c_int), ("sumsq_in", ctypes.c_void_p), ("parts", ctypes.c_int),
                ("width", ctypes.c_float), ("eps", ctypes.c_float)]


class NormEmit:
    """What an accumulate product is asked to leave for the RMS norm that reads its output
    rows next: `scaled` bf16 [rows, width] = bf16(x * gain), `sumsq` fp32 [parts, rows] = the
    tiles' shares of every row's sum of squares.  `parts` is set by the product that did it
    (None: it did not, the norm runs as a kernel of its own)."""

    def __init__(self, gain: torch.Tensor, scaled: torch.Tensor, sumsq: torch.Tensor, norm=None):
        self.gain, self.scaled, self.sumsq = gain, scaled, sumsq
        self.norm = norm              # the part the rows are left for (the caller's own reference)
        self.parts = None


def _norm_args(emit, pre, rows: int):
    """The pointer the product kernels take, and the object that keeps it alive."""
    if emit is None and pre is None:
        return _c_void_p(0), None
    args = _NormArgs()
    if emit is not None:
        args.gain, args.scaled = emit.gain.data_ptr(), emit.scaled.data_ptr()
        args.sumsq_out, args.ld_scaled = emit.sumsq.data_ptr(), emit.scaled.stride(0)
    if pre is not None:
        if pre.sumsq.stride(0) != rows or pre.sumsq.dtype != torch.float32:
            raise RuntimeError("shares of the rows' sums of squares must be float32 [parts, rows]")
        args.sumsq_in, args.parts = pre.sumsq.data_ptr(), pre.parts
        args.width, args.eps = float(pre.x.shape[1]), float(pre.eps)
    return ctypes.cast(ctypes.pointer(args), _c_void_p), args


def _gemm(a, w, out, n, epi, bn, per_sm=1, splits=None, emit=None, pre=None) -> bool:
    lib = build.load("gemm_tcgen05")
    if per_sm == 0:
        # 256 x 256 tiles; an output that cannot leave by TMA is refused, and the 128-row tiles run
        if _gemm(a, w, out, n, epi, 256, -1, 1, None, pre):
            return True
        per_sm = 1
    if per_sm == -1:
        per_sm, splits = 0, 1
    if splits is None:
        splits = k_splits(a.shape[0], 2 * n if epi == SWIGLU_BF16 else n, a.shape[1], bn)
    if emit is not None and (epi != ACCUM_F32 or bn > NORM_AHEAD_MAX_TILE or per_sm == 0 or n % 32
                             or emit.sumsq.shape[0] < -(-n // bn) or emit.sumsq.stride(0) != a.shape[0]):
        emit = None
    norm_ptr, keep = _norm_args(emit, pre, a.shape[0])
    code = lib.cb_gemm_tcgen05(
        _c_void_p(a.data_ptr()), _c_void_p(w.data_ptr()), _c_void_p(out.data_ptr()),
        _c_int(a.shape[0]), _c_int(n), _c_int(a.shape[1]), _c_int(a.stride(0)),
        _c_int(w.stride(0)), _c_int(out.stride(0)), _c_int(epi), _c_int(bn), _c_int(per_sm),
        _c_int(splits), _c_void_p(status_word(a.device).data_ptr()), _stream(), norm_ptr)
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"tensor-core matrix product failed to launch (CUDA error {code})")
    if emit is not None:
        emit.parts = -(-n // bn)
    _count(1)
    return True


_buffers = {}        # (device, name) -> tensor; grown by doubling, old ones kept alive because
_retired = []        # captured CUDA graphs may still hold their addresses


def _buffer(device, name: str, numel: int, dtype, zero: bool = False) -> torch.Tensor:
    key = (torch.device(device).index or 0, name)
    t = _buffers.get(key)
    if t is None or t.numel() < numel:
        if t is not None:
            _retired.append(t)
        make = torch.zeros if zero else torch.empty
        t = make(max(2 * numel, 1024), dtype=dtype, device=device)
        _buffers[key] = t
    return t


def skinny_splits(m: int, n_tiles: int, k: int) -> int:
    """Blocks along K per 128-row tile of W: as many as give every SM one block, never more
    blocks than SMs (a launch of at most one block per SM runs with eight stages, and every
    further split is a partial tile more for the last block to sum: 50 MB at 8 rows 13.7 us with
    3 x 48 blocks, 15.9 us with 4 x 48), and never so many that the partial tiles outweigh the
    weights they stand for."""
    k_blocks = -(-k // 64)
    want = max(1, N_SMS // n_tiles)
    cap = max(1, k // (4 * m))
    return max(1, min(want, k_blocks, cap))


def _gemm_skinny(a, w, out, n, epi, splits=None) -> bool:
    lib = build.load("gemm_skinny_tcgen05")
    m, k = a.shape
    n_tiles = int(lib.cb_gemm_skinny_tiles(_c_int(n), _c_int(epi)))
    if splits is None:
        splits = skinny_splits(m, n_tiles, k)
    partial = counters = None
    if splits > 1:
        lib.cb_gemm_skinny_partial_bytes.restype = ctypes.c_long
        nbytes = int(lib.cb_gemm_skinny_partial_bytes(_c_int(m), _c_int(n), _c_int(epi),
                                                      _c_int(splits)))
        partial = _buffer(a.device, "skinny.partial", nbytes // 4, torch.float32)
        counters = _buffer(a.device, "skinny.counters", n_tiles, torch.int32, zero=True)
    code = lib.cb_gemm_skinny(
        _c_void_p(a.data_ptr()), _c_void_p(w.data_ptr()), _c_void_p(out.data_ptr()),
        _c_int(m), _c_int(n), _c_int(k), _c_int(a.stride(0)), _c_int(w.stride(0)),
        _c_int(out.stride(0)), _c_int(epi), _c_int(splits),
        _c_void_p(partial.data_ptr() if partial is not None else 0),
        _c_void_p(counters.data_ptr() if counters is not None else 0),
        _c_void_p(status_word(a.device).data_ptr()), _stream())
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"tensor-core matrix product failed to launch (CUDA error {code})")
    _count(1)
    return True


SKINNY_ROWS = 16     # products with at most this many rows run with W on the MMA's M side ...
SKINNY_MIN_BYTES = 40 << 20   # ... if W is at least this large (it streams: 3.6-5.5 TB/s; smaller
                              # ones are latency-bound: at 33 MB and 16 rows the 128-row tiles, with
                              # K shared by clusters, take 12.7 us, these 12.4, the few-row kernel 12.1
                              # at 8 rows).
SKINNY_MID_ROWS = 32          # ... and up to this many rows between that size and SKINNY_MID_BYTES
SKINNY_MID_BYTES = 128 << 20  # (50 MB at 32 rows: 16.2 against 17.6 us for the tiles, 117 MB: 29.2
                              # against 33.3; 235 MB: 46.8 against 44.4).  From 33 rows on the
                              # 128-row tiles are as fast or faster at every size.
SKINNY_WIDE_N = 8192 # ... and up to 64 rows if W has at least this many rows (the LM head)


def _operands_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_cuda
            and a.stride(1) == 1 and w.stride(1) == 1 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear(a, w, out, *, accumulate=False, tile=None, emit=None, pre=None) -> bool:
    """`emit` (`NormEmit`): with accumulate, also leave the next norm's input if this product's
    form can (`emit.parts` says whether it did).  `pre` (`small_batch.LazyNorm` with `scaled`):
    `a` is that norm input, the rows' factors are applied in the epilogue."""
    if not _operands_ok(a, w) or out.stride(1) != 1:
        return False
    if out.dtype == torch.bfloat16:
        if accumulate:
            return False
        epi = STORE_BF16
    elif out.dtype == torch.float32:
        epi = ACCUM_F32 if accumulate else STORE_F32
    else:
        return False
    w_bytes = w.numel() * 2
    if tile is None and ((a.shape[0] <= SKINNY_ROWS and w_bytes >= SKINNY_MIN_BYTES)
                         or (a.shape[0] <= SKINNY_MID_ROWS and SKINNY_MIN_BYTES <= w_bytes <= SKINNY_MID_BYTES)
                         or (a.shape[0] <= 64 and w.shape[0] >= SKINNY_WIDE_N)):
        if pre is not None:
            return False
        return _gemm_skinny(a, w, out, w.shape[0], epi)
    if tile is None and _tall_tiles(a.shape[0], w.shape[0], a.shape[1]):
        tile = (256, 0)
    bn, per_sm, *splits = _tile_of(tile) if tile else _tile_width(a.shape[0], w.shape[0], epi)
    return _gemm(a, w, out, w.shape[0], epi, bn, per_sm, splits[0] if splits else None, emit, pre)


def linear_swiglu(h, gate_up, out, tile=None, pre=None) -> bool:
    if not _operands_ok(h, gate_up) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        return False
    inter = gate_up.shape[0] // 2
    if tile is None and h.shape[0] <= SKINNY_ROWS and gate_up.numel() * 2 >= SKINNY_MIN_BYTES:
        if pre is not None:
            return False
        return _gemm_skinny(h, gate_up, out, inter, SWIGLU_BF16)
    if tile is None and _tall_tiles(h.shape[0], 2 * inter, h.shape[1]):
        tile = (256, 0)
    bn, per_sm, *splits = _tile_of(tile) if tile else _tile_width(h.shape[0], 2 * inter, SWIGLU_BF16)
    return _gemm(h, gate_up, out, inter, SWIGLU_BF16, bn, per_sm, splits[0] if splits else None, None, pre)


ROPE_TALL = None     # tests may fix the form of the q/k/v product (True: 256 x 256 tiles)


def linear_rope_append(h, wqkv, qkv, n_heads, n_kv_heads, head_dim, cos, sin, rotary_dim, ctx, cache,
                       binding, pre=None) -> bool:
    """The q/k/v projection with the rotation and the cache write in the product's
    epilogue (whole head rotated, head size a multiple of 64).  Rotated q lands in the
    first columns of `qkv`; k and v only in the cache.  False: not taken."""
    if (not _operands_ok(h, wqkv) or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1
            or cos is None or rotary_dim != head_dim or head_dim % 64 or head_dim > 256
            or h.shape[0] <= SKINNY_ROWS):
        return False
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    if k_cache.dtype != torch.bfloat16:
        return False
    table = ctx.block_table(binding.group)
    bn, _ = _tile_width(h.shape[0], wqkv.shape[0], ROPE_APPEND, multiple_of=head_dim)
    tall = 256 % head_dim == 0 and _tall_tiles(h.shape[0], wqkv.shape[0], h.shape[1])
    if ROPE_TALL is not None:
        tall = ROPE_TALL
    if tall:
        bn = 256
    if bn % head_dim:
        return False
    lib = build.load("gemm_tcgen05")
    norm_ptr, keep = _norm_args(None, pre, h.shape[0])
    code = lib.cb_gemm_tcgen05_rope(
        _c_void_p(h.data_ptr()), _c_void_p(wqkv.data_ptr()), _c_void_p(qkv.data_ptr()),
        _c_int(h.shape[0]), _c_int(h.shape[1]), _c_int(h.stride(0)), _c_int(wqkv.stride(0)),
        _c_int(qkv.stride(0)), _c_int(bn), _c_void_p(cos.data_ptr()), _c_void_p(sin.data_ptr()),
        _c_void_p(ctx.positions.data_ptr()), _c_void_p(ctx.row_request.data_ptr()),
        _c_void_p(table.data_ptr()), _c_int(table.shape[1]), _c_void_p(k_cache.data_ptr()),
        _c_void_p(v_cache.data_ptr()), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim),
        _c_int(cache.page_tokens), _c_int(1 if binding.write else 0),
        _c_int(1 if tall else k_splits(h.shape[0], wqkv.shape[0], h.shape[1], bn)), _c_int(1 if tall else 0),
        _c_void_p(status_word(h.device).data_ptr()), _stream(), norm_ptr)
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"tensor-core q/k/v product failed to launch (CUDA error {code})")
    _count(1)
    return True


# The form of the head-size-64 prompt attention: -1 the launcher's choice (the roomy form, see the
# kernel's header), 0 roomy, 1 lean (tests fix it; CRUCIBLE_ATTENTION_LEAN=1 for a profile of that form).
ATTENTION_LEAN = int(os.environ.get("CRUCIBLE_ATTENTION_LEAN", "-1"))


class _Requests:
    """A run of consecutive requests of the step, as the attention kernels see one:
    the metadata arrays from its first request on, how many there are, the most new
    tokens any of them brings, the context bucket that covers them, and the number of
    the step's rows up to its end (the split form's scratch is indexed by row)."""

    def __init__(self, ctx, table, first: int, count: int, max_new: int, bucket: int, rows_end: int):
        self.row_start = ctx.req_row_start[first:]
        self.first_pos = ctx.req_first_pos[first:]
        self.table = table[first:]
        self.table_stride = table.shape[1]
        self.count, self.max_new, self.bucket, self.rows_end = count, max_new, bucket, rows_end


def _attention_tcgen05(qkv, out, k_cache, v_cache, reqs, n_heads, n_kv_heads, head_dim, scale,
                       window, cache) -> bool:
    """tcgen05 attention for portions of prompts: head size 64 or 128, page size a
    power of two from 8 to 128.  Returns False for anything else."""
    pt = cache.page_tokens
    if pt < 8 or pt > 128 or pt & (pt - 1):
        return False
    lib = build.load("attention_tcgen05")
    code = lib.cb_attention_tcgen05(
        _c_void_p(qkv.data_ptr()), _c_int(qkv.stride(0)), _c_void_p(out.data_ptr()),
        _c_int(out.stride(0)), _c_void_p(k_cache.data_ptr()), _c_void_p(v_cache.data_ptr()),
        _c_int(k_cache.shape[0]), _c_void_p(reqs.row_start.data_ptr()),
        _c_void_p(reqs.first_pos.data_ptr()), _c_void_p(reqs.table.data_ptr()),
        _c_int(reqs.table_stride), _c_int(reqs.count), _c_int(reqs.max_new),
        _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim), _c_int(pt),
        ctypes.c_float(scale), _c_int(window or 0), _c_int(ATTENTION_LEAN),
        _c_void_p(status_word(qkv.device).data_ptr()), _stream())
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"tcgen05 attention failed to launch (CUDA error {code})")
    _count(1)
    return True


def _attention_decode_tcgen05(qkv, out, k_cache, v_cache, reqs, n_heads, n_kv_heads, head_dim,
                              scale, window, cache, partial, counters, n_chunks,
                              chunk_keys) -> bool:
    """tcgen05 attention for decoded tokens (at most 16 packed rows per request and
    KV head): head size 64 or 128, page size a power of two from 8 to 128.  Returns False
    for anything else."""
    pt = cache.page_tokens
    if pt < 8 or pt > 128 or pt & (pt - 1):
        return False
    lib = build.load("attention_decode_tcgen05")
    code = lib.cb_attention_decode_tcgen05(
        _c_void_p(qkv.data_ptr()), _c_int(qkv.stride(0)), _c_void_p(out.data_ptr()),
        _c_int(out.stride(0)), _c_void_p(k_cache.data_ptr()), _c_void_p(v_cache.data_ptr()),
        _c_int(k_cache.shape[0]), _c_void_p(reqs.row_start.data_ptr()),
        _c_void_p(reqs.first_pos.data_ptr()), _c_void_p(reqs.table.data_ptr()),
        _c_int(reqs.table_stride), _c_int(reqs.count), _c_int(reqs.max_new),
        _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim), _c_int(pt),
        ctypes.c_float(scale), _c_int(window or 0), _c_void_p(partial.data_ptr()),
        _c_void_p(counters.data_ptr()), _c_int(n_chunks), _c_int(chunk_keys),
        _c_void_p(status_word(qkv.device).data_ptr()), _stream())
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"tcgen05 decode attention failed to launch (CUDA error {code})")
    _count(1)
    return True


DECODE_TC_TARGET_BLOCKS = 3 * N_SMS // 2  # two blocks of the tcgen05 decode kernel fit an SM, but they
                                          # start under the q/k/v product, whose blocks each take one
                                          # block's place until they end: a launch of more than about
                                          # one and a half blocks per SM starts in two waves
DECODE_TC_SHORT_BLOCKS = 22 * N_SMS // 10 # chunks of at most two tiles run with two K/V stages, three
                                          # blocks to an SM: a launch of up to this many finds its place
DECODE_MMA_TARGET_BLOCKS = 4 * N_SMS


def decode_chunk_keys(blocks_per_chunk: int, context_bucket: int, tcgen05: bool, head_dim: int = 64) -> int:
    """Keys per block of the split attention for decoded tokens: a function of the step's
    shape alone (so a captured step replays).  `blocks_per_chunk`: blocks that one chunk of
    every request takes (requests x KV heads x groups of 16 packed rows).  `context_bucket`:
    the longest context rounded up to a multiple of 256.

    tcgen05 form, from sweeps on B200 (120M shape, batch 1 to 64, contexts of 512 to 3,700):
    one tile of 128 keys per block while that is at most eight chunks (one round of the
    merge) and the launch finds its place at once; else two tiles per block while the launch
    finds its place (these short chunks run with two K/V stages, three blocks to an SM);
    else the bucket divided into as many equal parts as bring the launch nearest to one and
    a half blocks per SM, in whole tiles (batch 4 / 8 / 32 at 2,048 tokens: 0.307 / 0.321 /
    0.624 ms per step against 0.322 / 0.331 / 0.706 ms with chunks for 296 or 148 blocks).
    With heads of more than 64 features a block's three K/V stages are 192 KB, one block to an
    SM, and a launch of more blocks than SMs runs in two waves: the same rule with one block
    per SM as the most (Llama-3-8B layer sizes, 2,048 tokens, batch 4 / 8 / 16: 0.714 / 0.753 /
    0.824 ms per step of four layers against 0.736 / 0.773 / 0.854 ms).
    mma.sync form: the parts that bring the launch nearest to four blocks per SM."""
    unit = 128 if tcgen05 else 256
    whole = -(-context_bucket // unit) * unit
    one_per_sm = tcgen05 and head_dim > 64
    if tcgen05:
        short = N_SMS if one_per_sm else DECODE_TC_SHORT_BLOCKS
        n_one, n_two = -(-context_bucket // 128), -(-context_bucket // 256)
        if n_one <= 8 and blocks_per_chunk * n_one <= short:
            return min(128, whole)
        if blocks_per_chunk * n_two <= short:
            return min(256, whole)
    target = DECODE_TC_TARGET_BLOCKS if tcgen05 else DECODE_MMA_TARGET_BLOCKS
    if one_per_sm:
        parts = max(1, N_SMS // max(1, blocks_per_chunk))
    else:
        parts = max(1, (2 * target + blocks_per_chunk) // (2 * max(1, blocks_per_chunk)))
    chunk = -(-context_bucket // parts)
    chunk = -(-chunk // unit) * unit
    return min(max(chunk, unit), whole)


SPLIT_ROWS = 16          # packed rows (new tokens x heads of a group) the split form takes


def _attend(qkv, out, k_cache, v_cache, reqs, n_heads, n_kv_heads, head_dim, scale, window, ctx,
            cache) -> bool:
    """One run of requests through the kernel that suits it.  A function of the run's
    shape (count, most new tokens, bucket) and of the sizes only."""
    n_rep = n_heads // n_kv_heads
    split = reqs.max_new * n_rep <= SPLIT_ROWS
    pt = cache.page_tokens
    decode_tc = (USE_TCGEN05_DECODE and split and head_dim in (64, 128) and out.stride(0) % 2 == 0
                 and 8 <= pt <= 128 and pt & (pt - 1) == 0)
    partial = counters = None
    n_chunks, chunk_keys = 0, 256
    if split:
        groups = -(-reqs.max_new * n_rep // 16)
        blocks_per_chunk = reqs.count * n_kv_heads * groups
        chunk_keys = decode_chunk_keys(blocks_per_chunk, reqs.bucket, decode_tc, head_dim)
        n_chunks = -(-reqs.bucket // chunk_keys)
        floats = reqs.rows_end * n_heads * n_chunks * (head_dim + 2)
        partial = ctx.scratch("attn.partial", (floats,), torch.float32)
        counters = _buffer(qkv.device, "attn.counters", blocks_per_chunk, torch.int32, zero=True)
    if (decode_tc
            and _attention_decode_tcgen05(qkv, out, k_cache, v_cache, reqs, n_heads, n_kv_heads,
                                          head_dim, scale, window, cache, partial, counters,
                                          n_chunks, chunk_keys)):
        return True
    if (USE_TCGEN05_ATTENTION and not split and head_dim in (64, 128)
            and reqs.max_new * n_rep >= 64 and out.stride(0) % 8 == 0
            and _attention_tcgen05(qkv, out, k_cache, v_cache, reqs, n_heads, n_kv_heads,
                                   head_dim, scale, window, cache)):
        return True
    if split and chunk_keys % 256:
        # the mma.sync split form walks whole tiles of 256 keys
        chunk_keys = -(-chunk_keys // 256) * 256
        n_chunks = -(-reqs.bucket // chunk_keys)
    lib = build.load("attention_mma")
    code = lib.cb_attention_mma(
        _c_void_p(qkv.data_ptr()), _c_int(qkv.stride(0)), _c_void_p(out.data_ptr()),
        _c_int(out.stride(0)), _c_void_p(k_cache.data_ptr()), _c_void_p(v_cache.data_ptr()),
        _c_void_p(ctx.positions.data_ptr()), _c_void_p(reqs.row_start.data_ptr()),
        _c_void_p(reqs.first_pos.data_ptr()), _c_void_p(reqs.table.data_ptr()),
        _c_int(reqs.table_stride), _c_int(reqs.rows_end), _c_int(reqs.count),
        _c_int(reqs.max_new), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim),
        _c_int(cache.page_tokens), ctypes.c_float(scale), _c_int(window or 0),
        _c_void_p(partial.data_ptr() if partial is not None else 0),
        _c_void_p(counters.data_ptr() if counters is not None else 0), _c_int(n_chunks),
        _c_int(chunk_keys), _stream())
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"tensor-core attention failed to launch (CUDA error {code})")
    _count(1)
    return True


def paged_attention(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, ctx, cache,
                    binding) -> bool:
    """Tensor-core attention over the paged cache.  Takes head sizes that are
    multiples of 16 up to 256 and any head counts, group sizes and page sizes;
    refuses anything else (the plain kernel then runs).

    The kernel is chosen per request, not per step: requests that bring at most 16
    query rows per KV head (decoded tokens, tiny portions) run split over chunks of
    keys, with the last block of a row group to arrive merging; longer portions run as
    tiles (the tcgen05 kernel for head sizes 64 and 128, the mma.sync kernel of 64-row
    tiles else).  A step that holds both kinds (single decoded tokens first, as the
    scheduler orders them, then portions) is two launches over disjoint runs of its
    requests; the shapes of both are functions of the step's shape."""
    if (qkv.dtype != torch.bfloat16 or head_dim % 16 != 0 or head_dim > 256
            or n_heads % n_kv_heads != 0 or qkv.stride(0) % 8 != 0 or out.stride(0) % 2 != 0):
        return False
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    table = ctx.block_table(binding.group)
    host = ctx.host
    n_rep = n_heads // n_kv_heads
    args = (n_heads, n_kv_heads, head_dim, scale, window, ctx, cache)
    lead = host.lead_single
    if 0 < lead < ctx.n_requests and host.max_new_tokens * n_rep > SPLIT_ROWS:
        decoding = _Requests(ctx, table, 0, lead, 1, host.lead_context_bucket, lead)
        portions = _Requests(ctx, table, lead, ctx.n_requests - lead, host.max_new_tokens,
                             host.context_bucket, ctx.n_tokens)
        if not _attend(qkv, out, k_cache, v_cache, decoding, *args):
            return False
        if not _attend(qkv, out, k_cache, v_cache, portions, *args):
            raise RuntimeError("the attention kernels took the step's decoded tokens but "
                               "refused its portions: a rule of sizes is inconsistent")
        return True
    whole = _Requests(ctx, table, 0, ctx.n_requests, host.max_new_tokens, host.context_bucket,
                      ctx.n_tokens)
    return _attend(qkv, out, k_cache, v_cache, whole, *args)


def run_wait_probe(device, limit: int = 4096) -> None:
    """Launches a kernel whose only thread waits, bounded by `limit` polls, on a barrier
    nothing arrives at, and then records its give-up code in the status word: the failure
    path of the tensor-core kernels, made to happen without a fault (for tests)."""
    lib = build.load("gemm_tcgen05")
    code = lib.cb_tc_wait_probe(_c_void_p(status_word(device).data_ptr()), _c_int(limit), _stream())
    if code != 0:
        raise RuntimeError(f"wait probe failed to launch (CUDA error {code})")
