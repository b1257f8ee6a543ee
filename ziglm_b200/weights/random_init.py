"""Random weights from a configuration and a seed, in memory or as a model folder.

The reference's fixture generator fills every tensor from one seeded generator
with uniform values of +-0.01 and sets tensors whose name ends in ``norm.weight``
to 1 (src/synthetic.zig:232-249,430-447), and writes config.json and
model.safetensors with the architecture's own tensor names
(src/synthetic.zig:252-448).  Here values are N(0, std) with std 0.02 by
default; norm weights are 1, or 1 + N(0, norm_jitter) so that a test can tell a
norm's weight from its absence; each tensor has its own generator seeded from
(seed, tensor name), so a tensor's values do not depend on which others exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Mapping, Optional, Tuple

import torch

from ..parts.base import ParamDecl
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, decl: ParamDecl, seed: int, dtype: torch.dtype, device: torch.device,
                  std: float = 0.02, norm_jitter: float = 0.0) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if decl.kind == "int":
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    if decl.init == "ones":
        t = torch.ones(decl.shape, dtype=torch.float32, device=device)
        if norm_jitter:
            t += torch.randn(decl.shape, generator=gen, dtype=torch.float32, device=device) * norm_jitter
        return t.to(dtype)
    t = torch.randn(decl.shape, generator=gen, dtype=torch.float32, device=device) * std
    return t.to(dtype)


def random_tensors(declared: Mapping[str, ParamDecl], seed: int, dtype: torch.dtype, device: torch.device,
                   std: float = 0.02, norm_jitter: float = 0.0) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, decl in declared.items():
        yield name, random_tensor(name, decl, seed, dtype, device, std, norm_jitter)


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       norm_jitter: float = 0.0) -> None:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration)."""
    from ..engine.model import declare_parameters
    os.makedirs(folder, exist_ok=True)
    declared = declare_parameters(config.model_spec())
    tensors = dict(random_tensors(declared, seed, dtype, torch.device("cpu"), std, norm_jitter))
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
