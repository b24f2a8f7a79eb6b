"""Fused kernels for steps of a few rows (decoded tokens), bfloat16 engine only: up
to 32 rows, normalised bf16 input or fp32 rows with the norm inside.  Each
function returns True if it ran, False if the sizes are outside what the kernels
take (more rows, K not a multiple of 8, a partially rotated head, weights too
large to be worth it): the caller then runs the general kernels.

`LazyNorm` is what a norm part hands to a mixer or feed-forward that can fuse
the normalisation into its first matrix product: the fp32 rows, the gain and
eps, not yet normalised.  `tensor()` runs the norm kernel (once) for consumers
that need the normalised rows as a tensor.  For steps of many rows it may also
carry what the product that wrote the rows last left for the norm (`scaled`,
`sumsq`, `parts`: see `tensor_core.NormEmit`); a tensor-core product then takes
`scaled` as its rows and applies each row's factor in its epilogue.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Union

import torch

from . import build

build.register_module("decode_small", ["common.cuh"])

MAX_ROWS = 32           # rows these kernels take (in groups of 8)
PREFERRED_ROWS = 16     # rows up to which the callers choose them: measured on B200, a step of 17
                        # to 32 rows is as fast or faster through the 128-row tensor-core tiles
                        # (Llama-3.2-1B sizes at 32 rows: 9.7 against 13.1 us for q/k/v, 15.8
                        # against 48.5 us for gate/up)
MAX_LAZY_ROWS = 16      # rows a norm hands over not yet normalised: every block then normalises
                        # them for itself, which beyond 16 rows costs more than a norm kernel
_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_UNSUPPORTED = 100001


class LazyNorm:
    def __init__(self, x: torch.Tensor, gain: torch.Tensor, eps: float, materialize,
                 scaled: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None,
                 parts: int = 0):
        self.x, self.gain, self.eps = x, gain, eps
        self.scaled, self.sumsq, self.parts = scaled, sumsq, parts
        self._materialize = materialize
        self._tensor: Optional[torch.Tensor] = None
        self.shape = x.shape

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self._materialize()
        return self._tensor


Rows = Union[torch.Tensor, LazyNorm]


def as_tensor(h: Rows) -> torch.Tensor:
    return h.tensor() if isinstance(h, LazyNorm) else h


def _ptr(t):
    return _c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _input(h: Rows, w: torch.Tensor):
    """(x, gain, eps, a, lda) for the launchers."""
    if isinstance(h, LazyNorm) and (w.numel() * 2 > NORM_FUSE_MAX_BYTES or h.shape[0] > MAX_LAZY_ROWS):
        h = h.tensor()
    if isinstance(h, LazyNorm):
        if not h.x.is_contiguous():
            return None
        return h.x, h.gain, h.eps, None, 0
    if h.dtype != torch.bfloat16 or h.stride(1) != 1:
        return None
    return None, None, 0.0, h, h.stride(0)


def _done(code: int, what: str) -> bool:
    if code == _UNSUPPORTED:
        return False
    if code != 0:
        raise RuntimeError(f"{what} failed to launch (CUDA error {code})")
    from . import LAUNCHES
    LAUNCHES[0] += 1
    return True


# These kernels are built for latency (a few megabytes of weights per launch): 2.6-3.9 us
# for the 120M shape's matrices at 8 rows, where the 128-row tiles need 5.4-8.0 us.  They
# stream at 1.7 to 3.7 TB/s; the TMA-fed tensor-core kernel for few rows reaches 3.6 to
# 5.6 TB/s but costs a norm kernel and a reduction over K more (and for the q/k/v product a
# kernel for the rotation and the cache write).  Measured on B200 in replayed chains: at 34 MB
# the two are level (8 rows: 11.2-12.1 us here, 10.8-12.1 there), at 50 MB these take 18.0 us
# and that one 13.0, at 16 rows 24.2 against 13.9.
MAX_WEIGHT_BYTES = 40 << 20
MAX_WEIGHT_BYTES_TWO_GROUPS = 40 << 20
# Every block of a product normalises the step's rows for itself.  That is free while the
# blocks are few; with thousands of blocks it costs as much as the weights, and one norm
# kernel for all of them is cheaper.
NORM_FUSE_MAX_BYTES = 8 << 20


def _weights_ok(w: torch.Tensor, rows: int) -> bool:
    limit = MAX_WEIGHT_BYTES if rows <= 8 else MAX_WEIGHT_BYTES_TWO_GROUPS
    return (rows <= MAX_ROWS and w.dtype == torch.bfloat16 and w.is_cuda and w.stride(1) == 1
            and w.numel() * 2 <= limit)


MAX_OUT_ROWS = 8192     # wider products (the LM head) stream better through the tensor-core kernel


def linear(h: Rows, w: torch.Tensor, out: torch.Tensor, *, accumulate: bool = False) -> bool:
    if (not _weights_ok(w, h.shape[0]) or out.dtype != torch.float32 or out.stride(1) != 1
            or w.shape[0] > MAX_OUT_ROWS):
        return False
    inp = _input(h, w)
    if inp is None:
        return False
    x, gain, eps, a, lda = inp
    lib = build.load("decode_small")
    return _done(lib.cb_small_linear(_ptr(x), _ptr(gain), _c_float(eps), _ptr(a), _c_int(lda),
                                     _ptr(w), _c_int(w.stride(0)), _ptr(out), _c_int(out.stride(0)),
                                     _c_int(h.shape[0]), _c_int(w.shape[0]), _c_int(w.shape[1]),
                                     _c_int(1 if accumulate else 0), _stream()), "small linear")


def linear_swiglu(h: Rows, gate_up: torch.Tensor, out: torch.Tensor) -> bool:
    if (not _weights_ok(gate_up, h.shape[0]) or out.dtype != torch.bfloat16
            or out.stride(1) != 1):
        return False
    inp = _input(h, gate_up)
    if inp is None:
        return False
    x, gain, eps, a, lda = inp
    lib = build.load("decode_small")
    return _done(lib.cb_small_swiglu(_ptr(x), _ptr(gain), _c_float(eps), _ptr(a), _c_int(lda),
                                     _ptr(gate_up), _c_int(gate_up.stride(0)), _ptr(out),
                                     _c_int(out.stride(0)), _c_int(h.shape[0]),
                                     _c_int(gate_up.shape[0] // 2), _c_int(gate_up.shape[1]),
                                     _stream()), "small swiglu")


def qkv_rope_append(h: Rows, wqkv: torch.Tensor, qkv: torch.Tensor, n_heads: int, n_kv_heads: int,
                    head_dim: int, cos, sin, rotary_dim: int, ctx, cache, binding) -> bool:
    if (not _weights_ok(wqkv, h.shape[0]) or qkv.dtype != torch.bfloat16 or cos is None
            or rotary_dim != head_dim):
        return False
    inp = _input(h, wqkv)
    if inp is None:
        return False
    x, gain, eps, a, lda = inp
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    table = ctx.block_table(binding.group)
    lib = build.load("decode_small")
    return _done(lib.cb_small_qkv_rope_append(
        _ptr(x), _ptr(gain), _c_float(eps), _ptr(a), _c_int(lda), _ptr(wqkv),
        _c_int(wqkv.stride(0)), _ptr(qkv), _c_int(qkv.stride(0)), _ptr(cos), _ptr(sin),
        _c_int(rotary_dim), _ptr(ctx.positions), _ptr(ctx.row_request), _ptr(table),
        _c_int(table.shape[1]), _ptr(k_cache), _ptr(v_cache), _c_int(h.shape[0]),
        _c_int(wqkv.shape[1]), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim),
        _c_int(cache.page_tokens), _c_int(1 if binding.write else 0), _stream()),
        "small qkv + rope + cache write")
