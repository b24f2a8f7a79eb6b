"""Token embedding and LM head.

Embedding: x[t, :] = table[token[t], :], no scaling (`model.py:347`,
`engine/kernels/kernels.cu:1049-1059`); the gathered row is widened into the
fp32 residual stream; an id -(s + 1) stands for the token the engine last chose for
state slot s and is read on the device (`ctx.device_tokens`).  Head: logits = norm(x[rows]) W^T at the wanted rows only,
never [T, V] (`engine/src/gpu_model.rs:3590-3613`); W is the embedding table
when the model ties them (`model.py:289`), else its own matrix.  Logits are fp32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import EMBEDDINGS, HEADS, Embedding, Head, TensorDecl


class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, width: int):
        self.vocab_size = vocab_size
        self.width = width
        self.table = None

    def tensors(self):
        return [TensorDecl("table", (self.vocab_size, self.width))]

    def bind(self, tensors, dtype, device):
        self.table = tensors["table"]
        ops.declare_weights(self.table)

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        x = ctx.scratch("residual", (token_ids.shape[0], self.width), torch.float32)
        ops.embed_rows(self.table, token_ids, x, getattr(ctx, "device_tokens", None))
        return x


class LMHead(Head):
    def __init__(self, vocab_size: int, width: int, tied: bool):
        self.vocab_size = vocab_size
        self.width = width
        self.tied = tied
        self.weight = None

    def tensors(self):
        return [] if self.tied else [TensorDecl("weight", (self.vocab_size, self.width))]

    def bind(self, tensors, dtype, device):
        if not self.tied:
            self.weight = tensors["weight"]
            ops.declare_weights(self.weight)

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, ctx, normed_rows: torch.Tensor) -> torch.Tensor:
        logits = ctx.scratch("logits", (normed_rows.shape[0], self.vocab_size), torch.float32)
        ops.linear(normed_rows, self.weight, logits)
        return logits


EMBEDDINGS.register("token", lambda spec, vocab, width: TokenEmbedding(vocab, width))
HEADS.register("linear", lambda spec, vocab, width, tied: LMHead(vocab, width, tied))
