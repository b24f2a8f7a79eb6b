"""The operations the parts are written in, each a hand-written CUDA kernel.

Every function here launches on the current CUDA stream of torch and returns at
once.  Tensors are passed as raw device pointers through ctypes; shapes, dtypes
and contiguity are checked here, on the host, before anything is launched.
There is no CPU path: a tensor that is not on a CUDA device is an error, and so
is a kernel library that cannot be built or loaded.

Which kernel runs is decided by the engine dtype (float32: CUDA-core kernels
with fp32 arithmetic throughout; bfloat16: the tensor-core kernels, the fused
kernels for steps of a few rows, and the plain kernels as the stated refuge for
sizes the others do not take) and by the step's shape; every kernel computes
the same function, so a row's result depends on the path only by rounding.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_F32, _BF16 = 0, 1
_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("crucible_b200 kernels run on a CUDA device only; got a "
                              f"{t.device} tensor (there is no CPU path)")


def _contig(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


_scratch = {}       # per-device scratch of kernels that need some beyond inputs and outputs
LAUNCHES = [0]      # kernels launched through this module (graph replays add their own)


def _check(code: int, what: str) -> None:
    LAUNCHES[0] += 1
    if code != 0:
        lib = build.load("elementwise")
        lib.cb_error_string.restype = ctypes.c_char_p
        text = lib.cb_error_string(_c_int(code)).decode()
        raise KernelError(f"{what}: {text} (code {code})")


# ---------------------------------------------------------------------------
# row-wise kernels
# ---------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
               device_tokens: Optional[torch.Tensor] = None) -> None:
    """`device_tokens`: int32 per state slot; an id -(s + 1) reads device_tokens[s]."""
    _need_cuda(table, ids, out, device_tokens)
    if ids.dtype != torch.int32 or out.dtype != torch.float32:
        raise KernelError("embed_rows takes int32 ids and a float32 output")
    _contig(table, "embedding table"); _contig(out, "embed_rows output")
    lib = build.load("elementwise")
    _check(lib.cb_embed_rows(_ptr(table), _c_int(_code(table.dtype)), _ptr(ids), _ptr(out),
                             _c_int(ids.shape[0]), _c_int(table.shape[1]),
                             _c_int(table.shape[0]), _ptr(device_tokens), _stream()), "embed_rows")


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    _need_cuda(x, gain, out)
    if x.dtype != torch.float32 or gain.dtype != torch.float32:
        raise KernelError("rmsnorm takes a float32 input and a float32 gain")
    _contig(x, "rmsnorm input"); _contig(out, "rmsnorm output")
    lib = build.load("elementwise")
    _check(lib.cb_rmsnorm(_ptr(x), _ptr(gain), _ptr(out), _c_int(_code(out.dtype)),
                          _c_int(x.shape[0]), _c_int(x.shape[1]), _c_float(eps), _stream()),
           "rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(gate_up, out)
    if gate_up.dtype != out.dtype or gate_up.shape[1] != 2 * out.shape[1]:
        raise KernelError("swiglu takes [T, 2I] and writes [T, I] of the same dtype")
    _contig(gate_up, "swiglu input"); _contig(out, "swiglu output")
    lib = build.load("elementwise")
    _check(lib.cb_swiglu(_ptr(gate_up), _ptr(out), _c_int(_code(out.dtype)),
                         _c_int(out.shape[0]), _c_int(out.shape[1]), _stream()), "swiglu")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(x, rows, out)
    if x.dtype != torch.float32 or out.dtype != torch.float32 or rows.dtype != torch.int32:
        raise KernelError("gather_rows takes float32 rows and int32 indices")
    _contig(x, "gather_rows input"); _contig(out, "gather_rows output")
    lib = build.load("elementwise")
    _check(lib.cb_gather_rows(_ptr(x), _ptr(rows), _ptr(out), _c_int(out.shape[0]),
                              _c_int(x.shape[1]), _stream()), "gather_rows")


# ---------------------------------------------------------------------------
# matrix products: out[M, N] (+)= a[M, K] . w[N, K]^T
# ---------------------------------------------------------------------------

def linear_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *,
                 accumulate: bool = False) -> None:
    """The CUDA-core product: fp32 multiply-add, one ascending sum over k."""
    _need_cuda(a, w, out)
    if a.dtype != w.dtype or a.shape[1] != w.shape[1]:
        raise KernelError(f"linear: a is {tuple(a.shape)} {a.dtype}, w is {tuple(w.shape)} {w.dtype}")
    if out.shape[0] != a.shape[0] or out.shape[1] != w.shape[0]:
        raise KernelError(f"linear: output is {tuple(out.shape)}, expected "
                          f"{(a.shape[0], w.shape[0])}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("linear: accumulation goes into a float32 output")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear: rows must be contiguous")
    lib = build.load("gemm_simt")
    _check(lib.cb_gemm_simt(_ptr(a), _ptr(w), _ptr(out), _c_int(_code(a.dtype)),
                            _c_int(_code(out.dtype)), _c_int(a.shape[0]), _c_int(w.shape[0]),
                            _c_int(a.shape[1]), _c_int(a.stride(0)), _c_int(w.stride(0)),
                            _c_int(out.stride(0)), _c_int(1 if accumulate else 0), _stream()),
           "linear (CUDA cores)")


# Device ranges that hold weights: tensors that no kernel of a step writes.  The bfloat16
# product kernels ask for their matrix before the kernels ahead of them in the stream have
# finished (only the rows and the output wait for those), which is sound for a weight and a
# race for a matrix that an earlier kernel of the same step computes.  So a part declares
# its weights when it binds them, and a matrix that was not declared runs through the
# CUDA-core product, which reads nothing before its predecessors are done.
_weight_starts: list = []
_weight_ends: list = []


def declare_weights(*tensors: Optional[torch.Tensor]) -> None:
    """Says that these tensors are written by no kernel of any step, for as long as the
    tensor objects given here live (the declaration goes with them)."""
    import bisect
    import weakref
    for t in tensors:
        if t is None or not t.is_cuda:
            continue
        start = t.untyped_storage().data_ptr()
        end = start + t.untyped_storage().nbytes()
        at = bisect.bisect_left(_weight_starts, start)
        if at < len(_weight_starts) and _weight_starts[at] == start:
            continue
        _weight_starts.insert(at, start)
        _weight_ends.insert(at, end)
        weakref.finalize(t, _forget_weight, start)


def _forget_weight(start: int) -> None:
    import bisect
    at = bisect.bisect_left(_weight_starts, start)
    if at < len(_weight_starts) and _weight_starts[at] == start:
        del _weight_starts[at]
        del _weight_ends[at]


def is_weight(t: torch.Tensor) -> bool:
    import bisect
    p = t.data_ptr()
    at = bisect.bisect_right(_weight_starts, p) - 1
    return at >= 0 and p < _weight_ends[at]


def linear(a, w: torch.Tensor, out: torch.Tensor, *, accumulate: bool = False, closes=None) -> None:
    """`a` is a tensor or a `small_batch.LazyNorm` (rows not yet normalised).  `w`: if it was
    declared a weight (`declare_weights`) the bfloat16 kernels may fetch it early; any other
    matrix, one computed during the step for instance, takes the CUDA-core product.
    `closes`: the step's context, given by a part whose last write to the rows `out` this
    accumulating product is.  If the arrangement has announced the norm that reads those rows
    next (`StepContext.announce_norm`), the product may leave that norm's input beside its
    sums, and the norm then costs no kernel of its own."""
    from . import small_batch
    if w.dtype == torch.bfloat16 and is_weight(w):
        if a.shape[0] <= small_batch.PREFERRED_ROWS and small_batch.linear(a, w, out, accumulate=accumulate):
            return
        a = small_batch.as_tensor(a)
        from . import tensor_core
        emit = _norm_emit(closes, out, tensor_core) if accumulate and closes is not None else None
        if tensor_core.linear(a, w, out, accumulate=accumulate, emit=emit):
            if emit is not None and emit.parts:
                closes.offer_prenormed(out, emit.norm, emit.scaled, emit.sumsq, emit.parts)
            return
    a = small_batch.as_tensor(a)
    linear_plain(a, w, out, accumulate=accumulate)


def _norm_emit(ctx, rows: torch.Tensor, tensor_core):
    """What the accumulate product into `rows` may leave for the norm announced for them."""
    ahead = getattr(ctx, "norm_ahead", None)
    norm = ahead(rows) if ahead is not None and tensor_core.NORM_AHEAD else None
    if norm is None or rows.dtype != torch.float32 or not rows.is_contiguous():
        return None
    t, width = rows.shape
    scaled = ctx.scratch("norm.ahead.scaled", (t, width), torch.bfloat16)
    sumsq = ctx.scratch("norm.ahead.sumsq", (-(-width // 64), t), torch.float32)
    return tensor_core.NormEmit(norm.gain, scaled, sumsq, norm)


def _prenormed(h):
    """`h` if it carries a norm input that a product before it left, else None."""
    from . import small_batch
    return h if isinstance(h, small_batch.LazyNorm) and h.scaled is not None else None


def linear_swiglu(h, gate_up: torch.Tensor, out: torch.Tensor, ctx) -> None:
    """out[T, I] = silu(h Wg^T) * (h Wu^T) with gate_up = [Wg; Wu] of shape [2I, d]."""
    from . import small_batch
    if gate_up.dtype == torch.bfloat16 and is_weight(gate_up):
        if h.shape[0] <= small_batch.PREFERRED_ROWS and small_batch.linear_swiglu(h, gate_up, out):
            return
        from . import tensor_core
        pre = _prenormed(h)
        if pre is not None and tensor_core.linear_swiglu(pre.scaled, gate_up, out, pre=pre):
            return
        h = small_batch.as_tensor(h)
        if tensor_core.linear_swiglu(h, gate_up, out):
            return
    h = small_batch.as_tensor(h)
    both = ctx.scratch("ffn.gate_up", (h.shape[0], gate_up.shape[0]), h.dtype)
    linear(h, gate_up, both)
    swiglu(both, out)


def qkv_rope_append(h, wqkv: torch.Tensor, qkv: torch.Tensor, n_heads: int, n_kv_heads: int,
                    head_dim: int, cos, sin, rotary_dim: int, ctx, cache, binding) -> None:
    """The query/key/value projection, the rotation of q and k, and the write of
    k and v into the cache pages: one kernel for a few rows (mma.sync) and for many
    (tcgen05, rotation and cache write in the epilogue), two otherwise.  Leaves the
    rotated q in the first columns of `qkv`; the k and v columns of `qkv` are not
    defined afterwards (attention reads keys and values from the cache)."""
    from . import small_batch
    if not is_weight(wqkv):
        linear(h, wqkv, qkv)
        rope_kv_append(qkv, n_heads, n_kv_heads, head_dim, cos, sin, rotary_dim, ctx, cache, binding)
        return
    if (wqkv.dtype == torch.bfloat16 and h.shape[0] <= small_batch.PREFERRED_ROWS
            and small_batch.qkv_rope_append(h, wqkv, qkv, n_heads, n_kv_heads, head_dim, cos, sin,
                                            rotary_dim, ctx, cache, binding)):
        return
    if wqkv.dtype == torch.bfloat16 and h.shape[0] > small_batch.PREFERRED_ROWS:
        from . import tensor_core
        pre = _prenormed(h)
        if pre is not None and tensor_core.linear_rope_append(pre.scaled, wqkv, qkv, n_heads, n_kv_heads,
                                                              head_dim, cos, sin, rotary_dim, ctx, cache,
                                                              binding, pre=pre):
            return
        if tensor_core.linear_rope_append(small_batch.as_tensor(h), wqkv, qkv, n_heads, n_kv_heads,
                                          head_dim, cos, sin, rotary_dim, ctx, cache, binding):
            return
    linear(h, wqkv, qkv)
    rope_kv_append(qkv, n_heads, n_kv_heads, head_dim, cos, sin, rotary_dim, ctx, cache, binding)


# ---------------------------------------------------------------------------
# attention over the paged cache
# ---------------------------------------------------------------------------

def rope_kv_append(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                   ctx, cache, binding) -> None:
    _need_cuda(qkv)
    _contig(qkv, "qkv")
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope_kv_append: qkv width does not match the head counts")
    if rotary_dim:
        if cos is None or cos.shape[1] * 2 != rotary_dim or cos.dtype != torch.float32:
            raise KernelError("rope_kv_append: rotation tables must be float32 [positions, rotary_dim/2]")
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    if k_cache.dtype != qkv.dtype:
        raise KernelError("rope_kv_append: cache dtype differs from the activations'")
    table = ctx.block_table(binding.group)
    lib = build.load("elementwise")
    _check(lib.cb_rope_kv_append(
        _ptr(qkv), _c_int(_code(qkv.dtype)), _ptr(cos), _ptr(sin), _c_int(rotary_dim),
        _ptr(ctx.positions), _ptr(ctx.row_request), _ptr(table), _c_int(table.shape[1]),
        _ptr(k_cache), _ptr(v_cache), _c_int(qkv.shape[0]), _c_int(n_heads), _c_int(n_kv_heads),
        _c_int(head_dim), _c_int(cache.page_tokens), _c_int(1 if binding.write else 0),
        _stream()), "rope_kv_append")


def paged_attention_plain(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, ctx, cache,
                          binding) -> None:
    _need_cuda(qkv, out)
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    table = ctx.block_table(binding.group)
    lib = build.load("attention_generic")
    _check(lib.cb_attention_generic(
        _ptr(qkv), _c_int(qkv.stride(0)), _ptr(out), _c_int(out.stride(0)), _ptr(k_cache),
        _ptr(v_cache), _c_int(_code(qkv.dtype)), _ptr(ctx.positions), _ptr(ctx.row_request),
        _ptr(table), _c_int(table.shape[1]), _c_int(qkv.shape[0]), _c_int(n_heads),
        _c_int(n_kv_heads), _c_int(head_dim), _c_int(cache.page_tokens), _c_float(scale),
        _c_int(window or 0), _stream()), "paged attention (plain)")


def paged_attention(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, ctx, cache,
                    binding) -> None:
    if qkv.dtype == torch.bfloat16:
        from . import tensor_core
        if tensor_core.paged_attention(qkv, out, n_heads, n_kv_heads, head_dim, scale, window,
                                       ctx, cache, binding):
            return
    paged_attention_plain(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, ctx, cache,
                          binding)


# ---------------------------------------------------------------------------
# token selection
# ---------------------------------------------------------------------------

def _status_pair(status):
    """(source, destination) pointers of a status relay, or two nulls."""
    if status is None:
        return _c_void_p(0), _c_void_p(0)
    src, dst = status
    _need_cuda(src, dst)
    if src.dtype != torch.int32 or dst.dtype != torch.int32:
        raise KernelError("a status relay copies one int32 to another")
    return _ptr(src), _ptr(dst)


def argmax_rows(logits: torch.Tensor, out_ids: torch.Tensor,
                scatter_index: Optional[torch.Tensor] = None,
                scatter_out: Optional[torch.Tensor] = None, status=None) -> None:
    """`scatter_index`, `scatter_out` (int32): also write row r's id to
    scatter_out[scatter_index[r]].  `status`: (src, dst) int32 device tensors; the
    launch that writes the ids also copies src[0] to dst[0]."""
    _need_cuda(logits, out_ids, scatter_index, scatter_out)
    if logits.dtype != torch.float32 or out_ids.dtype != torch.int32:
        raise KernelError("argmax_rows takes float32 logits and int32 output")
    _contig(logits, "logits")
    lib = build.load("sampling")
    n = logits.shape[0]
    key = (logits.device.index, "argmax")
    scratch = _scratch.get(key)
    if scratch is None or scratch.numel() < n * 64:
        scratch = torch.empty(max(n, 64) * 64, dtype=torch.int32, device=logits.device)
        _scratch[key] = scratch
    # the rows' arrival counters of the one-launch form: zero between launches (the kernel puts
    # them back itself)
    counters = _scratch.get(key + ("counters",))
    if counters is None or counters.numel() < n:
        counters = torch.zeros(max(n, 1024), dtype=torch.int32, device=logits.device)
        _scratch[key + ("counters",)] = counters
    _check(lib.cb_argmax_rows(_ptr(logits), _c_int(n), _c_int(logits.shape[1]),
                              _ptr(out_ids), _ptr(scratch), _ptr(scatter_index), _ptr(scatter_out),
                              *_status_pair(status), _stream(), _ptr(counters)), "argmax_rows")


def max_device_top_k() -> int:
    return int(build.load("sampling").cb_sample_max_top_k())


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                uniform: torch.Tensor, max_top_k: int, out_ids: torch.Tensor,
                scatter_index: Optional[torch.Tensor] = None,
                scatter_out: Optional[torch.Tensor] = None, status=None) -> None:
    _need_cuda(logits, temperature, top_k, uniform, out_ids, scatter_index, scatter_out)
    if (logits.dtype != torch.float32 or temperature.dtype != torch.float32
            or uniform.dtype != torch.float32 or top_k.dtype != torch.int32
            or out_ids.dtype != torch.int32):
        raise KernelError("sample_rows: wrong tensor dtypes")
    _contig(logits, "logits")
    lib = build.load("sampling")
    code = lib.cb_sample_rows(_ptr(logits), _c_int(logits.shape[0]), _c_int(logits.shape[1]),
                              _ptr(temperature), _ptr(top_k), _ptr(uniform), _c_int(max_top_k),
                              _ptr(out_ids), _ptr(scatter_index), _ptr(scatter_out),
                              *_status_pair(status), _stream())
    if code == 100001:
        raise KernelError(f"top_k {max_top_k} exceeds what the sampling kernel holds "
                          f"({max_device_top_k()} candidates)")
    _check(code, "sample_rows")
