"""Dense gated feed-forward: down( act(gate(x)) * up(x) ), SwiGLU when act is silu.

The reference computes g = W_g x, u = W_u x, act_j = silu(g_j) u_j with
silu(z) = z/(1+exp(-z)), f = W_d act, no biases (src/model.zig:725-745,
src/math.zig:1108-1117; biases b_g, b_u, b_d are added to the three products when
the spec asks for them); its GPU path applies the tanh GELU to every
architecture (src/cuda_model.zig:695,1379), which is not reproduced.  Gate and
up are one matrix product over the concatenated weight [gate; up]; the
activation is a parameter of the part.  On the bfloat16 path the rows of that
weight alternate gate and up rows, so that the product's epilogue can apply the
activation and write act(gate) * up directly.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import FeedForwardSpec
from .base import NormedInput, ParamDecl, Part, register_feed_forward
from .linear import Linear


class GatedMLP(Part):
    def __init__(self, spec: FeedForwardSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        if spec.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated_mlp: activation {spec.activation!r} is not known (silu, gelu_tanh)")
        self.intermediate = spec.intermediate
        self.interleaved = False
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    @classmethod
    def declare(cls, spec: FeedForwardSpec) -> Dict[str, ParamDecl]:
        p = {"gate.weight": ParamDecl((spec.intermediate, spec.width)),
             "up.weight": ParamDecl((spec.intermediate, spec.width)),
             "down.weight": ParamDecl((spec.width, spec.intermediate))}
        if spec.bias:
            p["gate.bias"] = ParamDecl((spec.intermediate,))
            p["up.bias"] = ParamDecl((spec.intermediate,))
            p["down.bias"] = ParamDecl((spec.width,))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate.weight"], tensors["up.weight"]
        wide = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.interleaved = self.dtype == torch.bfloat16 and wide == torch.bfloat16
        bias = None
        if self.spec.bias:
            bg, bu = tensors["gate.bias"], tensors["up.bias"]
            bwide = torch.float32 if torch.float32 in (bg.dtype, bu.dtype) else bg.dtype
            parts = [bg.to(bwide), bu.to(bwide)]
            bias = torch.stack(parts, dim=1).reshape(-1) if self.interleaved else torch.cat(parts, dim=0)
        if self.interleaved:
            self.gate_up = Linear(torch.stack([g, u], dim=1).reshape(2 * self.intermediate, -1), bias)
        else:
            self.gate_up = Linear(torch.cat([g.to(wide), u.to(wide)], dim=0), bias)
        self.down = Linear(tensors["down.weight"], tensors["down.bias"] if self.spec.bias else None)

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("elementwise",)
        for lin in (self.gate_up, self.down):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    fuses_next_norm = True
    takes_normed_input = True

    def forward(self, step, h, residual: torch.Tensor, next_norm=None):
        """``h``: the normalised rows or a half-done norm (:class:`NormedInput`).  With ``next_norm`` the down
        projection may do the first half of that norm; the result is then its :class:`NormedInput`."""
        T = residual.shape[0]
        act = step.ws.buf("ffn_act", (T, self.intermediate), self.dtype)
        normed = isinstance(h, NormedInput)
        rows = h.hb if normed else h
        fused = self.interleaved and kernels.gemm_tc(rows, self.gate_up.weight, act, bias=self.gate_up.bias,
                                                     glu=self.spec.activation,
                                                     row_scale=(h.ssq, h.eps) if normed else None)
        if not fused:
            gu = step.ws.buf("gate_up", (T, 2 * self.intermediate), self.dtype)
            self.gate_up(h, gu)
            kernels.gated_act(gu, act, self.spec.activation, interleaved=self.interleaved)
        return self.down.accumulate_with_norm(step, act, residual, next_norm, "ffn_next")


register_feed_forward("gated_mlp", GatedMLP)
