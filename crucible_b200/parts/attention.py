"""Grouped-query attention over the paged cache.

q = n Wq^T, k = n Wk^T, v = n Wv^T; rotate q and k; write k, v at the token's
position in the request's pages; for a token at position p, keys j = lo..p
(lo = 0, or p - window + 1 with a window): s_j = (q . k_j) * scale,
softmax in fp32, o = sum_j p_j v_j; x += o Wo^T.  Query head h reads KV head
h // (n_heads // n_kv_heads) (division, not interleave).
`model.py:184-213`; `engine/src/model.rs:190-250`;
`engine/kernels/kernels.cu:1741-1839` (decode), `:1844-1925` (prefill).

The three projections are stored separately in the checkpoint
(`engine/src/model.rs:70-78`) and concatenated at load into one
[(Hq + 2 Hkv) * hd, d] operand.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.model_config import MixerSpec
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, TensorDecl


class PagedAttention(Mixer):
    fuses_norm = True

    def __init__(self, spec: MixerSpec):
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.head_dim <= 0:
            raise ValueError("attention needs positive n_heads, n_kv_heads and head_dim")
        if spec.n_heads % spec.n_kv_heads != 0:
            raise ValueError(f"n_heads ({spec.n_heads}) is not divisible by "
                             f"n_kv_heads ({spec.n_kv_heads})")
        if spec.window is not None and spec.window <= 0:
            raise ValueError(f"window must be positive, got {spec.window}")
        self.spec = spec
        self.position = (POSITIONS.build(spec.position.kind, spec.position)
                         if spec.position is not None else None)
        self.wqkv = None
        self.wo = None
        self.dtype = None

    @property
    def q_width(self):
        return self.spec.n_heads * self.spec.head_dim

    @property
    def kv_width(self):
        return self.spec.n_kv_heads * self.spec.head_dim

    def tensors(self):
        d = self.spec.width
        return [TensorDecl("q", (self.q_width, d)), TensorDecl("k", (self.kv_width, d)),
                TensorDecl("v", (self.kv_width, d)), TensorDecl("o", (d, self.q_width))]

    def bind(self, tensors, dtype, device):
        self.wqkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.wo = tensors["o"]
        ops.declare_weights(self.wqkv, self.wo)
        self.dtype = dtype
        if self.position is not None:
            self.position.bind({}, dtype, device)

    def cache_need(self):
        return CacheNeed(kv_heads=self.spec.n_kv_heads, head_dim=self.spec.head_dim,
                         window=self.spec.window)

    def forward(self, ctx, h, residual, binding):
        s = self.spec
        t = h.shape[0]
        qkv = ctx.scratch("attn.qkv", (t, self.q_width + 2 * self.kv_width), self.dtype)
        cache = ctx.cache(binding.group)
        rot = self.position.rotation() if self.position is not None else None
        if rot is not None or self.position is None:
            cos, sin, rotary_dim = rot if rot is not None else (None, None, 0)
            ops.qkv_rope_append(h, self.wqkv, qkv, s.n_heads, s.n_kv_heads, s.head_dim, cos, sin,
                                rotary_dim, ctx, cache, binding)
        else:
            # an encoding that is not a rotation: project, let it act on q and k,
            # then write k and v to the cache
            ops.linear(h, self.wqkv, qkv)
            q = qkv[:, :self.q_width].view(t, s.n_heads, s.head_dim)
            k = qkv[:, self.q_width:self.q_width + self.kv_width].view(t, s.n_kv_heads, s.head_dim)
            self.position.apply(ctx, q, k)
            ops.rope_kv_append(qkv, s.n_heads, s.n_kv_heads, s.head_dim, None, None, 0, ctx, cache,
                               binding)
        out = ctx.scratch("attn.out", (t, self.q_width), self.dtype)
        ops.paged_attention(qkv, out, s.n_heads, s.n_kv_heads, s.head_dim, s.softmax_scale,
                            s.window, ctx, cache, binding)
        ops.linear(out, self.wo, residual, accumulate=True, closes=ctx)


MIXERS.register("attention", PagedAttention)
