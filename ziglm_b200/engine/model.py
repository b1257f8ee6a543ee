"""The model: an embedding, blocks run in the order of the schedule, a final norm, a head; an architecture
may hang a part of its own behind the embedding and behind the head (``ModelSpec.embed_hook``, ``logits_hook``).

Built from a :class:`~ziglm_b200.config.spec.ModelSpec` alone.  The forward pass
is the reference's per-token loop (embedding src/model.zig:495-503, layers
543-789, final norm 794, head 797-802) over the packed tokens of a step: every
token of every sequence goes through the layers together, and the final norm and
head run only on the rows whose logits are wanted (the reference computes the
head for the last row of a chunk only, src/cuda_model.zig:1421-1434).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import ModelSpec
from ..parts import Linear, ParamDecl, block_class, hook_class, norm_class
from ..parts.base import KVNeed, StateNeed
from .batch import StepContext


def declare_parameters(spec: ModelSpec) -> Dict[str, ParamDecl]:
    """Every tensor the model owns, by the name it has in the weight files.  Touches no device."""
    out: Dict[str, ParamDecl] = {spec.embedding_name: ParamDecl((spec.vocab_size, spec.width))}
    for layer in spec.layers:
        for local, decl in block_class(layer.block).declare(layer).items():
            out[layer.prefix + layer.names.get(local, local)] = decl
    for local, decl in norm_class(spec.final_norm.kind).declare(spec.final_norm).items():
        out[_final_norm_name(spec, local)] = decl
    if spec.head_name is not None:
        out[spec.head_name] = ParamDecl((spec.vocab_size, spec.width))
    for hook in (spec.embed_hook, spec.logits_hook):
        if hook is not None:
            for local, decl in hook_class(hook.kind).declare(hook).items():
                out[hook.names.get(local, local)] = decl
    return out


def _final_norm_name(spec: ModelSpec, local: str) -> str:
    base = spec.final_norm_name
    return base if local == "weight" else base.rsplit(".", 1)[0] + "." + local


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the model runs in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.blocks = [block_class(layer.block)(layer, dtype, device) for layer in spec.layers]
        self.final_norm = norm_class(spec.final_norm.kind)(spec.final_norm, dtype, device)
        self.embed_hook = hook_class(spec.embed_hook.kind)(spec.embed_hook, dtype, device) if spec.embed_hook else None
        self.logits_hook = hook_class(spec.logits_hook.kind)(spec.logits_hook, dtype, device) if spec.logits_hook else None
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None

    # ------------------------------------------------------------------ weights
    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (already on the device, already checked against declare_parameters)."""
        spec = self.spec
        self.embedding = tensors[spec.embedding_name].contiguous()
        for layer, block in zip(spec.layers, self.blocks):
            local = {}
            for name in block_class(layer.block).declare(layer):
                local[name] = tensors[layer.prefix + layer.names.get(name, name)]
            block.bind(local)
        self.final_norm.bind({name: tensors[_final_norm_name(spec, name)]
                              for name in norm_class(spec.final_norm.kind).declare(spec.final_norm)})
        head_weight = self.embedding if spec.head_name is None else tensors[spec.head_name]
        self.head = Linear(head_weight)
        for hook_spec, hook in ((spec.embed_hook, self.embed_hook), (spec.logits_hook, self.logits_hook)):
            if hook is not None:
                hook.bind({local: tensors[hook_spec.names.get(local, local)]
                           for local in hook_class(hook_spec.kind).declare(hook_spec)})

    def kernel_libraries(self) -> Tuple[str, ...]:
        libs = ("elementwise",) + self.final_norm.kernel_libraries()
        for b in self.blocks:
            libs += b.kernel_libraries()
        if self.head is not None:
            libs += self.head.libraries(self.dtype)
        for hook in (self.embed_hook, self.logits_hook):
            if hook is not None:
                libs += hook.kernel_libraries()
        return tuple(dict.fromkeys(libs))

    # ----------------------------------------------------- what the cache must hold
    def cache_plan(self) -> Tuple[List[Optional[KVNeed]], List[Optional[int]], List[Optional[StateNeed]]]:
        """Per place of the schedule: keys/values kept, the place read instead, fixed state kept."""
        kv: List[Optional[KVNeed]] = []
        reads: List[Optional[int]] = []
        state: List[Optional[StateNeed]] = []
        last_place_of: Dict[int, int] = {}
        for place, li in enumerate(self.spec.schedule):
            block = self.blocks[li]
            src_layer = self.spec.layers[li].mixer.cache_from
            if src_layer is not None:
                if src_layer not in last_place_of:
                    raise ValueError(f"layer {li} reads the cache of layer {src_layer}, which has not run before it")
                kv.append(None)
                reads.append(last_place_of[src_layer])
            else:
                kv.append(block.cache_needs())
                reads.append(None)
            state.append(block.state_needs())
            last_place_of[li] = place
        return kv, reads, state

    # ------------------------------------------------------------------ forward
    def forward(self, step: StepContext) -> Optional[torch.Tensor]:
        """Run the step's tokens through the layers; float32 logits [n_want, vocab] or None."""
        spec = self.spec
        x = step.ws.buf("residual", (step.n_tokens, spec.width), torch.float32)
        kernels.embed(self.embedding, step.tokens, x, spec.embedding_scale)
        if self.embed_hook is not None:
            self.embed_hook.forward(step, x)
        carried = None           # the next block's first norm, half done by the block before (steps of few tokens)
        for place, li in enumerate(spec.schedule):
            block = self.blocks[li]
            nxt = self.blocks[spec.schedule[place + 1]] if place + 1 < len(spec.schedule) else None
            takes = getattr(nxt, "accepts_normed_input", None)
            next_norm = nxt.mixer_norm if takes is not None and takes() else None
            if carried is not None or next_norm is not None:
                carried = block.forward(step, step.io[place], x, h_in=carried, next_norm=next_norm)
            else:
                block.forward(step, step.io[place], x)
        if step.n_want == 0:
            return None
        h = self.final_norm.forward(step, x, rows=step.want_rows, n_rows=step.n_want, name="final_norm_out")
        logits = step.ws.buf("logits", (step.n_want, spec.vocab_size), torch.float32)
        self.head(h, logits)
        if self.logits_hook is not None:
            self.logits_hook.forward(step, logits)
        return logits
