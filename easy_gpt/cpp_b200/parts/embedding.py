"""Token embedding and the output head.

Embedding: residual[t] = E[id[t]] (src/models/embedding.cpp:54-76).  Head:
logits = x E^T when tied (the reference always is, src/models/gpt_model.cpp:324-328,
src/models/embedding.cpp:78-81) or x W_head^T with ``lm_head.weight`` when not.
Logits are float32 in both precisions.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import Part, PendingNorm
from .linear import Linear


class TokenEmbedding(Part):
    capturable = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.table = None

    def tensor_requests(self):
        return [TensorRequest.matrix(self.prefix + ".weight", self.vocab, self.hidden)]

    def load(self, tensors, device, dtype):
        self.table = tensors[self.prefix + ".weight"].to(device=device, dtype=dtype).contiguous()

    def forward(self, ctx, residual):
        """residual[t] = table[ctx.token_ids[t]] for the step's tokens (float32 [T, hidden])."""
        kernels.embedding_gather(ctx.token_ids, self.table, residual, ctx.status)


class LMHead(Part):
    """params: vocab_size, hidden_size, tied_to (prefix of the embedding, or None)."""

    capturable = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.linear = None

    def tensor_requests(self):
        if self.tied_to:
            return []
        return [TensorRequest.matrix(self.prefix + ".weight", self.vocab, self.hidden)]

    def load(self, tensors, device, dtype, tied_table=None):
        if self.tied_to:
            self.linear = Linear.sharing(tied_table)
        else:
            self.linear = Linear(tensors[self.prefix + ".weight"], None, device, dtype)

    def weight_bytes(self):
        return self.linear.weight_bytes()

    def streamed_weights(self):
        # the head is far larger than the L2; only its first rows are worth asking for ahead of time
        rows = min(self.vocab, (24 << 20) // (self.hidden * self.linear.weight.element_size()))
        return [self.linear.weight[:rows]]

    accepts_pending_norm = True
    # Thousands of CTAs share the head's rows, and each would repeat the add + norm of the few tokens in front of its
    # product: normalising once in a kernel of its own measured 1.7% faster per decode step at batch 8.
    fuse_norm = False

    def forward(self, x, status=None):
        """x: normalised rows [R, hidden] or a PendingNorm; returns float32 logits [R, vocab]."""
        if isinstance(x, PendingNorm):
            if x.fusable and self.fuse_norm:
                out = torch.empty((x.residual.shape[0], self.vocab), device=x.residual.device, dtype=torch.float32)
                kernels.gemm_skinny(self.linear.weight, None, out, kernels.EPI_F32, norm=x.fused())
                return out
            x = x.materialize()
        return self.linear(x, out_dtype=torch.float32, status=status)


register_part("head", "embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
