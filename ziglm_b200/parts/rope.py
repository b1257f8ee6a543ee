"""Rotary position encoding: the table of inverse frequencies and the rules that stretch it.

A head's first ``rotary_dim`` elements are rotated in pairs (i, i + rotary_dim/2)
by the angle pos * inv_freq[i] (src/model.zig:569-597; the reference supports
rotary_dim < head_dim at src/model.zig:571-572).  The reference derives the
frequency as 1/powf(base, 2i/rot) inside the kernel with a base it picks from
the head size (src/cuda_bridge.cu:2070-2108, src/model.zig:405-413); here
inv_freq[i] = theta^(-2i/rot) comes from the configuration, is computed once in
float64 and rounded to float32, and the angle is formed in float32.

Scaling rules, each applied once to the table (``rope_type`` of the configuration's ``rope_scaling``):

linear (position interpolation): f_i / factor.

llama3: with wavelength l_i = 2*pi/f_i and L0 = original_max_position_embeddings,
    l_i < L0/high_freq_factor : f_i stays
    l_i > L0/low_freq_factor  : f_i / factor
    otherwise                 : s = (L0/l_i - low)/(high - low);
                                f_i <- (1-s) * f_i/factor + s * f_i

yarn: the pair index at which a frequency makes r rotations over L0 positions is
    d(r) = rot * ln(L0 / (2 pi r)) / (2 ln theta);
with lo = d(beta_fast), hi = d(beta_slow) (rounded down and up unless ``truncate`` is false, and kept inside
[0, rot-1]; hi is raised by 0.001 if it equals lo), g_i = clamp((i - lo)/(hi - lo), 0, 1):
    f_i <- (1 - g_i) * f_i + g_i * f_i / factor
so pairs that turn fast keep their frequency and slow ones are interpolated.  The rule also multiplies the
rotated queries and keys by ``attention_factor`` (default 0.1 ln(factor) + 1); since the whole head is
rotated, that is the same as multiplying the scores by its square, which is what ``score_scale`` reports
to the mixer.
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional, Tuple

import torch

from ..config.spec import PositionSpec
from .base import Part, register_position


def scaling_kind(scaling: Optional[Mapping[str, Any]]) -> Optional[str]:
    if not scaling:
        return None
    kind = scaling.get("rope_type", scaling.get("type"))
    return None if kind in (None, "default") else kind


def inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[Mapping[str, Any]]) -> torch.Tensor:
    """float32 [rotary_dim/2], computed in float64."""
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be positive and even, found {rotary_dim}")
    idx = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inv = torch.exp(-(idx / rotary_dim) * math.log(theta))
    kind = scaling_kind(scaling)
    if kind is None:
        pass
    elif kind == "linear":
        inv = inv / float(scaling["factor"])
    elif kind == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        mixed = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, mixed))
    elif kind == "yarn":
        factor = float(scaling["factor"])
        orig = float(scaling["original_max_position_embeddings"])
        fast = float(scaling.get("beta_fast") or 32.0)
        slow = float(scaling.get("beta_slow") or 1.0)

        def pair_of(rotations: float) -> float:
            return rotary_dim * math.log(orig / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))

        lo, hi = pair_of(fast), pair_of(slow)
        if scaling.get("truncate", True) is not False:
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rotary_dim - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float64) - lo) / (hi - lo)).clamp(0.0, 1.0)
        inv = (1.0 - ramp) * inv + ramp * inv / factor
    else:
        raise ValueError(f"rope scaling of type {kind!r} is not supported (linear, llama3, yarn)")
    return inv.to(torch.float32)


def score_factor(scaling: Optional[Mapping[str, Any]]) -> float:
    """What the rule multiplies queries and keys by (1 for every rule but yarn)."""
    if scaling_kind(scaling) != "yarn":
        return 1.0
    given = scaling.get("attention_factor")
    if given is not None:
        return float(given)
    factor = float(scaling["factor"])
    return 1.0 if factor <= 1.0 else 0.1 * math.log(factor) + 1.0


class Rope(Part):
    def __init__(self, spec: PositionSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.rotary_dim = spec.rotary_dim
        self.inv_freq = inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling).to(device)
        self.factor = score_factor(spec.scaling)

    def score_scale(self, head_dim: int) -> float:
        """What the mixer multiplies its scores by on behalf of this encoding."""
        if self.factor != 1.0 and head_dim != self.rotary_dim:
            raise ValueError("a rope scaling that scales queries and keys needs the whole head to be rotated "
                             f"(rotary_dim {self.rotary_dim}, head size {head_dim})")
        return self.factor * self.factor

    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.rotary_dim

    def apply(self, step, qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError("rotary positions are applied by the cache-write kernel")


class NoPosition(Part):
    """No position information enters the mixer."""

    def rotary_table(self):
        return None

    def score_scale(self, head_dim: int) -> float:
        return 1.0

    def apply(self, step, qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
