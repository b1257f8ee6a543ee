"""Rotary position encoding: the table of inverse frequencies and its llama3 scaling.

A head's first ``rotary_dim`` elements are rotated in pairs (i, i + rotary_dim/2)
by the angle pos * inv_freq[i] (src/model.zig:569-597; the reference supports
rotary_dim < head_dim at src/model.zig:571-572).  The reference derives the
frequency as 1/powf(base, 2i/rot) inside the kernel with a base it picks from
the head size (src/cuda_bridge.cu:2070-2108, src/model.zig:405-413); here
inv_freq[i] = theta^(-2i/rot) comes from the configuration, is computed once in
float64 and rounded to float32, and the angle is formed in float32.

llama3 scaling, applied once to the table: with wavelength l_i = 2*pi/f_i and
L0 = original_max_position_embeddings,
    l_i < L0/high_freq_factor : f_i stays
    l_i > L0/low_freq_factor  : f_i / factor
    otherwise                 : s = (L0/l_i - low)/(high - low);
                                f_i <- (1-s) * f_i/factor + s * f_i
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional, Tuple

import torch

from ..config.spec import PositionSpec
from .base import Part, register_position


def inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[Mapping[str, Any]]) -> torch.Tensor:
    """float32 [rotary_dim/2], computed in float64."""
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be positive and even, found {rotary_dim}")
    idx = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inv = torch.exp(-(idx / rotary_dim) * math.log(theta))
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind != "llama3":
            raise ValueError(f"rope scaling of type {kind!r} is not supported (only 'llama3')")
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        mixed = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, mixed))
    return inv.to(torch.float32)


class Rope(Part):
    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.rotary_dim = spec.rotary_dim
        self.inv_freq = inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling).to(device)

    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.rotary_dim

    def apply(self, step, qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError("rotary positions are applied by the cache-write kernel")


class NoPosition(Part):
    """No position information enters the mixer."""

    def rotary_table(self):
        return None

    def apply(self, step, qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
