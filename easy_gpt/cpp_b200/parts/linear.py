"""y = x W^T + b with W stored [out, in] (src/models/linear.cpp:42-44).

In bfloat16, steps of up to 64 tokens (decoding) go to the package's own
weight-streaming kernel (``csrc/gemm_skinny.cu``); larger ones go to the library
GEMM (cuBLAS through torch), where the reference's engine calls cublasGemmEx too
(src/cuda/ops/matmul.cu:194-204).  In float32 it is always the
package's own FFMA kernel: true 32-bit arithmetic whose sums do not depend on
the batch.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], device, dtype: torch.dtype):
        self.weight = weight.to(device=device, dtype=dtype).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.dtype = dtype
        # the bias is added in float32 by our kernels; the library GEMM wants it in its own dtype
        self.bias_f32 = None if bias is None else bias.to(device=device, dtype=torch.float32).reshape(-1).contiguous()
        self.bias = None if bias is None else self.bias_f32.to(dtype)

    @classmethod
    def sharing(cls, weight: torch.Tensor) -> "Linear":
        """A bias-free product with a weight that another part owns (a tied head
        multiplies by the embedding table itself, not by a copy)."""
        self = cls.__new__(cls)
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        self.dtype = weight.dtype
        self.bias = self.bias_f32 = None
        return self

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def takes_following_norm(self, x: torch.Tensor) -> bool:
        """Whether ``with_following_norm`` can run for this input (the decode kernel takes it)."""
        return (self.dtype == torch.bfloat16 and kernels.gemm_skinny_takes(self.dtype, x.shape[0], self.in_features)
                and x.shape[0] <= kernels.FUSED_NORM_MAX_TOKENS and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)

    def with_following_norm(self, x: torch.Tensor, follow, prefetch: Optional[torch.Tensor] = None,
                            status: Optional[torch.Tensor] = None):
        """The product, the add to the residual and the preparation of the norm that follows, in one
        kernel: follow.residual += x W^T + b (in place); returns a PreNormed for follow.norm."""
        from .base import PreNormed
        rows, ss_parts = kernels.gemm_skinny(self.weight, self.bias_f32, None, kernels.EPI_RESID_NORM, x=x, prefetch=prefetch,
                                             status=status, follow=dict(residual=follow.residual, gain=follow.gain))
        return PreNormed(follow.norm, rows, ss_parts)

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 prefetch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``status``: the step's status word; with it the tcgen05 product for 17..128 rows may run
        (its bounded waits report there)."""
        M = x.shape[0]
        out_dtype = out_dtype or self.dtype
        if self.dtype == torch.float32:
            out = torch.empty((M, self.out_features), device=x.device, dtype=torch.float32)
            kernels.gemm_f32_nt(x, self.weight, self.bias_f32, out)
            return out
        if kernels.gemm_skinny_takes(self.dtype, M, self.in_features) and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
            out = torch.empty((M, self.out_features), device=x.device, dtype=out_dtype)
            kernels.gemm_skinny(self.weight, self.bias_f32, out,
                                kernels.EPI_F32 if out_dtype == torch.float32 else kernels.EPI_STORE, x=x, prefetch=prefetch)
            return out
        if (status is not None and kernels.gemm_tcgen05_few_takes(self.dtype, M, self.out_features, self.in_features)
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and x.stride(1) == 1):
            out = torch.empty((M, self.out_features), device=x.device, dtype=out_dtype)
            kernels.gemm_tcgen05_few(x, self.weight, self.bias_f32, out, status,
                                     epilogue=kernels.EPI_F32 if out_dtype == torch.float32 else kernels.EPI_STORE)
            return out
        if out_dtype == torch.float32:
            out = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
            if self.bias_f32 is not None:
                out += self.bias_f32
            return out
        return torch.nn.functional.linear(x, self.weight, self.bias)
