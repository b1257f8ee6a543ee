"""Grouped-query attention with rotary positions over the paged cache.

Order of operations, as in the reference's layer loop (src/model.zig:557-706;
GPU twin src/cuda_model.zig:1255-1352): q, k, v projections of the normed input,
rotation of q and k by position, k and v written to the cache (keys stored
rotated), per head softmax(q.K^T * scale) V over the keys the token may see
(all earlier ones, or a window), output projection, sum into the residual.
Query head h reads key/value head h // (n_heads // n_kv_heads)
(src/model.zig:554).  The reference has no biases; q/k/v/o biases are added to
the projections when the spec asks for them.

The three input projections are one matrix product over the concatenated weight
[q; k; v] (the reference runs three, src/cuda_model.zig:1265,1294-1298, and fuses
them only for one quantized format).  A layer whose spec names ``cache_from``
owns no k and v projections: it rotates its queries and reads the other layer's
keys and values (the reference's shared-KV layers, src/model.zig:599-618).
"""
from __future__ import annotations

import math
import warnings
from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import MixerSpec
from .base import KVNeed, LayerIO, ParamDecl, Part, StateNeed, position_class, register_mixer
from .linear import Linear


_warned = set()      # (head size, group) pairs whose slow path has been announced


class Attention(Part):
    def __init__(self, spec: MixerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} heads cannot share {spec.n_kv_heads} key/value heads")
        if spec.head_dim % 8 or spec.head_dim > 256:
            raise ValueError(f"attention: head size {spec.head_dim} is not supported (a multiple of 8, at most 256)")
        self.n_heads, self.n_kv, self.head_dim = spec.n_heads, spec.n_kv_heads, spec.head_dim
        self.shares_cache = spec.cache_from is not None
        self.scale = float(spec.scale) if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.window = spec.window
        self.position = position_class(spec.position.kind)(spec.position, dtype, device)
        score_scale = getattr(self.position, "score_scale", None)
        if score_scale is not None:
            self.scale *= float(score_scale(spec.head_dim))
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        if dtype == torch.bfloat16 and not kernels.fast_attention_libraries(dtype, spec.head_dim, spec.n_heads,
                                                                            spec.n_kv_heads):
            key = (spec.head_dim, spec.n_heads // spec.n_kv_heads)
            if key not in _warned:
                _warned.add(key)
                warnings.warn(
                    f"attention with head size {spec.head_dim} and {key[1]} query heads per key/value head runs on the "
                    "plain CUDA-core kernel, which is right but many times slower than the tensor-core kernels "
                    "(those take head sizes 64 and 128 with at most 16 query heads per key/value head)",
                    RuntimeWarning, stacklevel=2)

    @classmethod
    def declare(cls, spec: MixerSpec) -> Dict[str, ParamDecl]:
        q, kv, d = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim, spec.width
        p = {"q.weight": ParamDecl((q, d)), "o.weight": ParamDecl((d, q))}
        if spec.cache_from is None:
            p["k.weight"] = ParamDecl((kv, d))
            p["v.weight"] = ParamDecl((kv, d))
        if spec.bias:
            p["q.bias"] = ParamDecl((q,))
            if spec.cache_from is None:
                p["k.bias"] = ParamDecl((kv,))
                p["v.bias"] = ParamDecl((kv,))
        if spec.out_bias:
            p["o.bias"] = ParamDecl((d,))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        names = ["q"] if self.shares_cache else ["q", "k", "v"]
        ws = [tensors[f"{n}.weight"] for n in names]
        wide = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        weight = torch.cat([w.to(wide) for w in ws], dim=0)
        bias = None
        if self.spec.bias:
            bs = [tensors[f"{n}.bias"] for n in names]
            bwide = torch.float32 if any(b.dtype == torch.float32 for b in bs) else bs[0].dtype
            bias = torch.cat([b.to(bwide) for b in bs], dim=0)
        self.qkv = Linear(weight, bias)
        self.o = Linear(tensors["o.weight"], tensors.get("o.bias") if self.spec.out_bias else None)

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("attention",) + kernels.fast_attention_libraries(self.dtype, self.head_dim, self.n_heads, self.n_kv)
        for lin in (self.qkv, self.o):
            if lin is not None:
                libs += lin.libraries(self.dtype)
        return libs

    def cache_needs(self) -> Optional[KVNeed]:
        if self.shares_cache:
            return None
        return KVNeed(self.n_kv, self.head_dim, self.window)

    def state_needs(self) -> Optional[StateNeed]:
        return None

    fuses_next_norm = True
    takes_normed_input = True

    def forward(self, step, io: LayerIO, h, residual: torch.Tensor, next_norm=None):
        """``h``: the normalised rows or a half-done norm (:class:`NormedInput`).  With ``next_norm`` the output
        projection may do the first half of that norm; the result is then its :class:`NormedInput`."""
        T = residual.shape[0]
        n_kv_here = 0 if self.shares_cache else self.n_kv
        qkv = step.ws.buf("qkv", (T, (self.n_heads + 2 * n_kv_here) * self.head_dim), self.dtype)
        self.qkv(h, qkv)
        table = self.position.rotary_table()
        if table is None:
            self.position.apply(step, qkv, self.n_heads, n_kv_here, self.head_dim)
            inv_freq, rot = None, 0
        else:
            inv_freq, rot = table
        store = io.writes_cache and not self.shares_cache
        out = step.ws.buf("attn_out", (T, self.n_heads * self.head_dim), self.dtype)
        if kernels.attention_with_rope(step, qkv, out, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window,
                                       io, inv_freq, rot, store):
            return self.o.accumulate_with_norm(step, out, residual, next_norm, "attn_next")
        kernels.rope_store(qkv, self.n_heads, n_kv_here, self.head_dim, rot, inv_freq, step.positions,
                           step.seq_of_token, io.block_table, io.k_pages if store else None,
                           io.v_pages if store else None, io.page_size)
        kernels.attention(step, qkv, out, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window, io)
        return self.o.accumulate_with_norm(step, out, residual, next_norm, "attn_next")


register_mixer("attention", Attention)
