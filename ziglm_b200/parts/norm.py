"""RMSNorm: y_i = x_i / sqrt(mean(x^2) + eps) * w_i, statistics in float32.

The reference computes ``ss = sum x^2; inv = 1/sqrt(ss/n + eps); y = (x*inv)*w``
(src/math.zig:850-945, src/cuda_bridge.cu:1475-1534) and adds 1 to the weight
only for Gemma (src/types.zig:279-283); that offset is the ``unit_offset`` option
here and is off unless a spec asks for it.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import NormSpec
from .base import ParamDecl, Part, register_norm


class RMSNorm(Part):
    fusable = True

    def __init__(self, spec: NormSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.width = spec.width
        self.eps = float(spec.eps)
        self.weight_offset = 1.0 if spec.options.get("unit_offset") else 0.0
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def declare(cls, spec: NormSpec) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((spec.width,), init="ones")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def kernel_libraries(self) -> Tuple[str, ...]:
        return ("elementwise",)

    def forward(self, step, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                name: str = "norm_out") -> torch.Tensor:
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        if out is None:
            out = step.ws.buf(name, (n, self.width), self.dtype)
        kernels.rmsnorm(x, self.weight, out, self.eps, rows=rows, weight_offset=self.weight_offset)
        return out


register_norm("rmsnorm", RMSNorm)
