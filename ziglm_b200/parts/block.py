"""The pre-norm residual arrangement: x += mixer(norm(x)); x += ffn(norm(x)).

This is the reference's layer body for the architectures without post-norms:
norm, attention, residual sum, norm, feed-forward, residual sum
(src/model.zig:545-546,704-716,719-755).  The residual stream x is float32 in
both precisions; mixers and feed-forwards add into it themselves, so the sum
rides in the epilogue of their last matrix product.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.spec import LayerSpec
from .base import (KVNeed, LayerIO, ParamDecl, Part, StateNeed, feed_forward_class, mixer_class, norm_class,
                   register_block)


class PreNormBlock(Part):
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        super().__init__(spec, dtype, device)
        self.mixer_norm = norm_class(spec.mixer_norm.kind)(spec.mixer_norm, dtype, device)
        self.mixer = mixer_class(spec.mixer.kind)(spec.mixer, dtype, device)
        self.ffn_norm = norm_class(spec.ffn_norm.kind)(spec.ffn_norm, dtype, device)
        self.ffn = feed_forward_class(spec.ffn.kind)(spec.ffn, dtype, device)

    @classmethod
    def _children(cls, spec: LayerSpec):
        return (("mixer_norm.", norm_class(spec.mixer_norm.kind), spec.mixer_norm),
                ("mixer.", mixer_class(spec.mixer.kind), spec.mixer),
                ("ffn_norm.", norm_class(spec.ffn_norm.kind), spec.ffn_norm),
                ("ffn.", feed_forward_class(spec.ffn.kind), spec.ffn))

    @classmethod
    def declare(cls, spec: LayerSpec) -> Dict[str, ParamDecl]:
        out: Dict[str, ParamDecl] = {}
        for prefix, klass, sub in cls._children(spec):
            for name, decl in klass.declare(sub).items():
                out[prefix + name] = decl
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in (("mixer_norm.", self.mixer_norm), ("mixer.", self.mixer),
                             ("ffn_norm.", self.ffn_norm), ("ffn.", self.ffn)):
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        return (self.mixer_norm.kernel_libraries() + self.mixer.kernel_libraries()
                + self.ffn_norm.kernel_libraries() + self.ffn.kernel_libraries())

    def cache_needs(self) -> Optional[KVNeed]:
        return self.mixer.cache_needs()

    def state_needs(self) -> Optional[StateNeed]:
        return self.mixer.state_needs()

    def accepts_normed_input(self) -> bool:
        """Whether ``forward`` may be handed this block's first norm half done (``h_in``)."""
        return bool(self.mixer_norm.fusable and self.mixer.takes_normed_input)

    def forward(self, step, io: LayerIO, x: torch.Tensor, h_in=None, next_norm=None):
        """``h_in``: this block's first norm, half done by the block before (else the norm kernel runs).
        ``next_norm``: the first norm of the block after; the result is its half-done form if the feed-forward's
        last product did it, else None."""
        h = h_in if h_in is not None else self.mixer_norm.forward(step, x)
        if self.mixer.fuses_next_norm and self.ffn.takes_normed_input and self.ffn_norm.fusable:
            h = self.mixer.forward(step, io, h, x, next_norm=self.ffn_norm)
        else:
            self.mixer.forward(step, io, h, x)
            h = None
        if h is None:
            h = self.ffn_norm.forward(step, x)
        if self.ffn.fuses_next_norm and next_norm is not None:
            return self.ffn.forward(step, h, x, next_norm=next_norm)
        self.ffn.forward(step, h, x)
        return None


register_block("prenorm", PreNormBlock)
