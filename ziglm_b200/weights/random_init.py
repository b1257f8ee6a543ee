"""Random weights from a configuration and a seed, in memory or as a model folder.

The reference's fixture generator fills every tensor from one seeded generator
with uniform values of +-0.01 and sets tensors whose name ends in ``norm.weight``
to 1 (src/synthetic.zig:232-249,430-447), and writes config.json and
model.safetensors with the architecture's own tensor names
(src/synthetic.zig:252-448).  Here values are N(0, std) with std 0.02 by
default; norm weights are 1, or 1 + N(0, norm_jitter) so that a test can tell a
norm's weight from its absence.

Every value is a function of (seed, tensor name, element index) alone: a tensor's
key is a hash of seed and name, and element i is the Box-Muller value of the two
24-bit numbers in mix64(key + i).  The arithmetic is a fixed list of single
IEEE-rounded float32 operations (ln, sin and cos are short polynomials), so the
device kernel (``zlm_fill_normal`` in csrc/elementwise.cu) and NumPy
(:func:`normal_values`) give the same bits.  A model made on the device by
``Engine.from_config`` therefore holds exactly the tensors that
``write_random_model`` writes for the same configuration and seed, and any slice
of any tensor can be regenerated without the rest.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Mapping, Optional, Tuple

import numpy as np
import torch

from ..parts.base import ParamDecl
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's values."""
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def _mix64(x: np.ndarray) -> np.ndarray:
    x = x + np.uint64(0x9E3779B97F4A7C15)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def _poly(x2: np.ndarray, coefficients) -> np.ndarray:
    f = np.float32
    p = np.full_like(x2, f(coefficients[0]))
    for c in coefficients[1:]:
        p = p * x2 + f(c)          # two roundings: NumPy does not fuse
    return p


def normal_values(key: int, start: int, count: int) -> np.ndarray:
    """Standard normal values of elements ``start .. start+count`` of the tensor with this key, float32.

    h = mix64(key + i); u1 = (top 24 bits + 1) / 2^24; angle = 2 pi (next 24 bits) / 2^24;
    z = sqrt(-2 ln u1) cos(angle).  ln u1 = (e - 24) ln 2 + ln m with u1 2^24 = m 2^e, m in (sqrt(1/2), sqrt(2)],
    ln m = 2 s (1 + s^2/3 + s^4/5 + s^6/7 + s^8/9), s = (m - 1)/(m + 1); the cosine is taken by octants with
    the argument folded into [0, pi/4] and the Taylor polynomials to x^9 (sine) and x^10 (cosine)."""
    f = np.float32
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        h = _mix64(np.uint64(key & _M64) + idx)
    n = ((h >> np.uint64(40)) + np.uint64(1)).astype(np.uint32)
    b = ((h >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.uint32)
    mant, exp = np.frexp(n.astype(f))                    # n = mant 2^exp, mant in [1/2, 1): exact
    m = mant * f(2.0)
    e = exp.astype(np.int32) - 1
    big = m > f(1.41421354)
    m = np.where(big, m * f(0.5), m)
    e = np.where(big, e + 1, e)
    s = (m + f(-1.0)) / (m + f(1.0))
    s2 = s * s
    p = _poly(s2, (1.11111111e-1, 1.42857143e-1, 0.2, 3.33333333e-1, 1.0))
    ln_m = (f(2.0) * s) * p
    ln_u = (e - 24).astype(f) * f(0.693147182) + ln_m
    r = np.sqrt(f(-2.0) * ln_u)
    octant = b >> np.uint32(21)
    rem = b & np.uint32(0x1FFFFF)
    folded = np.where(octant & np.uint32(1), np.uint32(0x200000) - rem, rem)
    x = folded.astype(f) * f(3.74507039e-7)
    x2 = x * x
    sin = x * _poly(x2, (2.75573192e-6, -1.98412698e-4, 8.33333333e-3, -1.66666667e-1, 1.0))
    cos = _poly(x2, (-2.75573192e-7, 2.48015873e-5, -1.38888889e-3, 4.16666667e-2, -0.5, 1.0))
    use_sin = ((octant + np.uint32(1)) >> np.uint32(1)) & np.uint32(1) != 0          # octants 1, 2, 5, 6
    negative = ((octant + np.uint32(2)) >> np.uint32(2)) & np.uint32(1) != 0         # octants 2, 3, 4, 5
    c = np.where(use_sin, sin, cos)
    c = np.where(negative, -c, c)
    return (r * c).astype(f)


_CHUNK = 1 << 14         # the temporaries of a chunk stay in the cache of the CPU


def _fill_cpu(shape, key: int, mean: float, std: float, dtype: torch.dtype) -> torch.Tensor:
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=dtype)
    f = np.float32
    for start in range(0, n, _CHUNK):
        count = min(_CHUNK, n - start)
        v = f(mean) + f(std) * normal_values(key, start, count)
        out[start:start + count] = torch.from_numpy(v).to(dtype)         # bfloat16: round to nearest even
    return out.view(*shape)


def random_tensor(name: str, decl: ParamDecl, seed: int, dtype: torch.dtype, device: torch.device,
                  std: float = 0.02, norm_jitter: float = 0.0) -> torch.Tensor:
    """The tensor ``name`` of a random model: the same values on the device (a kernel) and on the CPU (NumPy)."""
    device = torch.device(device)
    if decl.kind == "int":
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    if decl.init == "ones":
        mean, spread = 1.0, float(norm_jitter)
    else:
        mean, spread = 0.0, float(std)
    if spread == 0.0:
        return torch.full(decl.shape, mean, dtype=dtype, device=device)
    key = tensor_key(seed, name)
    if device.type == "cuda":
        from .. import kernels
        out = torch.empty(decl.shape, dtype=dtype, device=device)
        with torch.cuda.device(device):
            kernels.fill_normal(out, key, mean, spread)
        return out
    return _fill_cpu(decl.shape, key, mean, spread, dtype)


def random_tensors(declared: Mapping[str, ParamDecl], seed: int, dtype: torch.dtype, device: torch.device,
                   std: float = 0.02, norm_jitter: float = 0.0) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, decl in declared.items():
        yield name, random_tensor(name, decl, seed, dtype, device, std, norm_jitter)


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       norm_jitter: float = 0.0, device: Optional[torch.device] = None) -> None:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration).  ``device``: where
    the values are computed before they are written (default: the CPU; a CUDA device gives the same file faster)."""
    from ..engine.model import declare_parameters
    os.makedirs(folder, exist_ok=True)
    declared = declare_parameters(config.model_spec())
    made = random_tensors(declared, seed, dtype, torch.device(device or "cpu"), std, norm_jitter)
    tensors = {name: t.cpu() for name, t in made}
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
