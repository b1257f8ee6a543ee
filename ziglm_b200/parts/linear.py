"""y = x W^T (+ bias): picks the matrix-product kernel for the operand types and the row count.

The weight is [out_features, in_features], as the files store it and as the
reference multiplies it (y[r] = sum_c W[r,c] x[c], src/math.zig:730-758,
src/cuda_bridge.cu:963-1018).  float32 operands go to the CUDA-core product
(the true 32-bit path).  bfloat16 operands go to the tensor-core kernels: a
weight-streaming kernel for the few rows of a decode step and the tcgen05/TMA
kernel for prompts; sizes those kernels refuse fall back to the CUDA-core
product, never to a wrong result.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import NormedInput


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("a linear weight must be a matrix")
        self.weight = weight.contiguous()
        self.bias = bias.contiguous() if bias is not None else None
        self.out_features, self.in_features = self.weight.shape
        self._fast = None   # prepared state of the tensor-core kernels, built on first use

    def libraries(self, dtype: torch.dtype):
        if dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            return ("gemm_generic",) + kernels.fast_gemm_libraries()
        return ("gemm_generic",)

    def __call__(self, x, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
        """``x``: the input rows, or a :class:`NormedInput` whose norm this product completes."""
        if isinstance(x, NormedInput):
            if x.hb.shape[-1] != self.in_features:
                raise ValueError(f"linear: input width {x.hb.shape[-1]} does not match the weight's {self.in_features}")
            if not kernels.fast_gemm(self, x.hb, out, accumulate, row_scale=(x.ssq, x.eps)):
                raise kernels.KernelError("linear: a half-done norm reached a product the tensor-core kernel refuses")
            return out
        if x.shape[-1] != self.in_features:
            raise ValueError(f"linear: input width {x.shape[-1]} does not match the weight's {self.in_features}")
        if kernels.fast_gemm(self, x, out, accumulate):
            return out
        kernels.gemm_generic(x, self.weight, out, bias=self.bias, accumulate=accumulate)
        return out

    def accumulate_with_norm(self, step, x: torch.Tensor, residual: torch.Tensor, norm, name: str) -> Optional[NormedInput]:
        """residual += x W^T (+ bias); if the step is small enough for the product to finish every element of
        the residual in one thread, it also does the first half of ``norm`` (an RMSNorm part) and the result
        says so; else None (the caller runs the norm kernel)."""
        T, d = residual.shape
        if (norm is None or not norm.fusable or T > 64 or x.dtype != torch.bfloat16
                or self.weight.dtype != torch.bfloat16 or residual.dtype != torch.float32):
            self(x, residual, accumulate=True)
            return None
        hb = step.ws.buf(name + "_hb", (T, d), torch.bfloat16)
        ssq = step.ws.buf(name + "_ssq", (T, -(-d // 128)), torch.float32)
        done = kernels.fast_gemm(self, x, residual, True, norm_out=(norm.weight, norm.weight_offset, hb, ssq))
        if not done:
            kernels.gemm_generic(x, self.weight, residual, bias=self.bias, accumulate=True)
            return None
        return NormedInput(hb, ssq, norm.eps) if done == 2 else None
