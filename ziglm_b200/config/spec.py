"""Architecture-neutral description of a decoder: what each layer is made of.

A model is data: a list of :class:`LayerSpec` (one per set of weights) and a
``schedule`` that says in which order the layers run.  The schedule may name a
layer twice, and a mixer may read another layer's cache (``cache_from``).
Every size and constant a part needs is carried here, so that no part has to
know which model it is in.  An architecture's typed configuration (for
instance :class:`ziglm_b200.config.llama.LlamaConfig`) produces a
:class:`ModelSpec`; the engine only ever sees the spec.

The reference keeps the same per-layer quantities on its ``LayerWeights``
(src/model.zig:38-50: head_dim, n_heads, n_kv_heads, rope_theta, rotary_dim,
sliding_window, intermediate_size) but branches on a global architecture enum in
the forward pass (src/model.zig:500,635,659,736); here the branch is replaced by
the ``kind`` strings below, resolved through the part registries.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the model width."""
    kind: str                      # registry key, e.g. "rmsnorm"
    width: int
    eps: float
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer (rotary tables, nothing, ...)."""
    kind: str                      # registry key, e.g. "rope", "none"
    rotary_dim: int = 0
    theta: float = 10000.0
    scaling: Optional[Mapping[str, Any]] = None
    max_positions: int = 0
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class MixerSpec:
    """The token mixer of a layer (attention here)."""
    kind: str                      # registry key, e.g. "attention"
    width: int                     # model width d
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    bias: bool = False
    out_bias: bool = False
    window: Optional[int] = None   # None: every earlier key is visible
    scale: Optional[float] = None  # None: 1/sqrt(head_dim)
    position: PositionSpec = PositionSpec(kind="none")
    cache_from: Optional[int] = None   # read (and do not write) this layer's cache
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class FeedForwardSpec:
    """The per-token feed-forward of a layer (dense gated MLP here)."""
    kind: str                      # registry key, e.g. "gated_mlp"
    width: int
    intermediate: int
    activation: str = "silu"
    bias: bool = False
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One set of layer weights and how its parts are arranged.

    ``options`` carries what an arrangement other than the pre-norm one needs beyond the four parts: further
    part specs (a norm after the mixer, say) or scalars, under names the arrangement defines.  The pre-norm
    arrangement reads none."""
    block: str                     # registry key of the arrangement, e.g. "prenorm"
    prefix: str                    # tensor-name prefix of this layer's weights
    mixer_norm: NormSpec
    mixer: MixerSpec
    ffn_norm: NormSpec
    ffn: FeedForwardSpec
    # local parameter name (as the part declares it) -> name under ``prefix``
    names: Mapping[str, str] = field(default_factory=dict)
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class HookSpec:
    """A part that runs once per step outside the layers: on the embedded tokens before the first layer
    (learned absolute positions, an embedding norm) or on the logits after the head (a bias, a soft cap)."""
    kind: str                      # registry key
    options: Mapping[str, Any] = field(default_factory=dict)
    # local parameter name (as the part declares it) -> full tensor name in the weight files
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    width: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[int, ...]      # indices into ``layers`` in running order
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    head_name: Optional[str]       # None: the head is the embedding table (tied)
    embedding_scale: float = 1.0
    max_positions: int = 0
    stop_token_ids: Tuple[int, ...] = ()
    embed_hook: Optional[HookSpec] = None      # runs on the float32 residual [T, width] after the embedding
    logits_hook: Optional[HookSpec] = None     # runs on the float32 logits [n_want, vocab] after the head
    options: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        for i in self.schedule:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"schedule names layer {i}, but there are {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            src = layer.mixer.cache_from
            if src is not None and not 0 <= src < len(self.layers):
                raise ValueError(f"layer {i} reads the cache of layer {src}, which does not exist")
