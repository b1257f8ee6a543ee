"""What every part of a layer has in common, and the registries that find parts by kind.

A part is built from its spec alone (sizes and constants are parameters; no part
knows which model it is in), declares the tensors it owns under local names,
is handed those tensors on the device, and runs on a step.

Interfaces
----------
Norm            ``forward(step, x, out=None, rows=None) -> out``: x is the float32
                residual stream [T, d]; the result has the step's storage type.
PositionEncoding``rotary_table() -> (inv_freq, rotary_dim) | None`` for encodings
                that are a rotation by position (fused into the cache write), and
                ``apply(step, qkv, n_heads, n_kv_heads, head_dim)`` for any other.
Mixer           ``cache_needs() -> KVNeed | None``, ``state_needs() -> StateNeed |
                None``, ``forward(step, io, h, residual)``: adds its output to the
                float32 ``residual`` in place.  ``io`` is the storage of the place
                in the schedule that is running (:class:`LayerIO`).
FeedForward     ``forward(step, h, residual)``: adds its output to ``residual``.
Block           ``forward(step, io, x)``: runs its parts on the residual stream x.
Hook            ``forward(step, x)``: changes x in place; x is the float32 residual
                [T, d] after the embedding (``ModelSpec.embed_hook``) or the float32
                logits [n_want, vocab] (``ModelSpec.logits_hook``).

A norm that rides on its neighbours
-----------------------------------
In steps of a few tokens a norm kernel between two matrix products costs more in
waiting than in work, so a part may offer to do the norm that follows it, and a
part may accept its input normalised that way:
``fuses_next_norm``   the part's ``forward`` takes ``next_norm=<norm part>`` and
                      returns a :class:`NormedInput` if its last product did the
                      norm's first half (x * gain and the sums of squares), else None;
``takes_normed_input``the part's ``forward`` takes a :class:`NormedInput` in place
                      of ``h`` and completes the norm in its first product.
``fusable``           (norms) the norm is gain * x / sqrt(mean x^2 + eps) and nothing else.
Parts without these attributes are never asked; a block falls back to the norm kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamDecl:
    """A tensor a part owns: its shape, whether it is a table of integers, how random weights fill it."""
    shape: Tuple[int, ...]
    kind: str = "float"            # "float" or "int"
    init: str = "normal"           # "normal" (N(0, std)) or "ones" (norm weights)


@dataclass(frozen=True)
class KVNeed:
    """Keys and values a mixer wants kept: per position n_kv_heads x head_dim, all of them or a window."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state a mixer wants kept per sequence (zero when the sequence starts)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerIO:
    """Storage of one place in the schedule for the running step."""
    k_pages: Optional[torch.Tensor] = None      # [n_pages, n_kv, page_size, head_dim]
    v_pages: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None  # int32 [B, stride], rows in batch order
    page_size: int = 0
    writes_cache: bool = True
    state: Optional[torch.Tensor] = None        # [n_slots, *shape]; index with step.slots


@dataclass
class NormedInput:
    """A norm's input half done: ``hb`` [T, d] holds bf16(x * gain), ``ssq`` [T, P] float32 partial sums of
    x^2 (summed over P they give the row's sum of squares).  The product that reads ``hb`` multiplies its
    output rows by 1 / sqrt(sum(ssq[t]) / d + eps)."""
    hb: torch.Tensor
    ssq: torch.Tensor
    eps: float


class Part:
    """Base of all parts."""
    fuses_next_norm = False
    takes_normed_input = False
    fusable = False

    def __init__(self, spec: Any, dtype: torch.dtype, device: torch.device):
        self.spec = spec
        self.dtype = dtype
        self.device = device

    @classmethod
    def declare(cls, spec: Any) -> Dict[str, ParamDecl]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def kernel_libraries(self) -> Tuple[str, ...]:
        """Names of the CUDA sources this part launches kernels from."""
        return ()


_REGISTRIES: Dict[str, Dict[str, Any]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
                                          "hook": {}}


def _register(family: str, kind: str, cls: Any) -> None:
    table = _REGISTRIES[family]
    if kind in table and table[kind] is not cls:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    table[kind] = cls


def _lookup(family: str, kind: str) -> Any:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise KeyError(f"no {family} of kind {kind!r} is registered (known: {known})") from None


def register_norm(kind: str, cls: Any) -> None: _register("norm", kind, cls)
def register_position(kind: str, cls: Any) -> None: _register("position", kind, cls)
def register_mixer(kind: str, cls: Any) -> None: _register("mixer", kind, cls)
def register_feed_forward(kind: str, cls: Any) -> None: _register("feed_forward", kind, cls)
def register_block(kind: str, cls: Any) -> None: _register("block", kind, cls)
def register_hook(kind: str, cls: Any) -> None: _register("hook", kind, cls)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def norm_class(kind: str) -> Any: return _lookup("norm", kind)
def position_class(kind: str) -> Any: return _lookup("position", kind)
def mixer_class(kind: str) -> Any: return _lookup("mixer", kind)
def feed_forward_class(kind: str) -> Any: return _lookup("feed_forward", kind)
def block_class(kind: str) -> Any: return _lookup("block", kind)
def hook_class(kind: str) -> Any: return _lookup("hook", kind)
