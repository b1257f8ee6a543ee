"""Binds the tensors of a model folder to the names a model declares.

Everything that is wrong with a folder's tensors is reported in one
:class:`WeightError`: names the model needs that the files lack, names the files
hold that the model does not know, and shapes or kinds that disagree.  The
reference requires only the embedding and the final norm and silently skips any
other missing tensor in its forward pass (src/model.zig:302-304 and the
``if (layer.attn_q) |t|`` tests at 557,621,704,728-745); nothing is skipped here.

Storage types: with ``dtype=bfloat16`` floating tensors are kept in bfloat16,
except that a tensor the file stores in 32-bit stays float32; with
``dtype=float32`` every floating tensor is widened to float32 (exact for
bfloat16 and float16 sources).  Integer tables become int32.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..parts.base import ParamDecl
from .safetensors_io import SafetensorsError, open_model_files

# Buffers some exporters write that are not parameters of any part.
IGNORED_TENSORS = ("*.rotary_emb.inv_freq",)

_FLOATS = {"F32", "BF16", "F16", "F64"}
_INTS = {"I64", "I32", "I16", "I8", "U8"}


class WeightError(ValueError):
    """The tensors of a model folder do not match what the model declares."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"the tensors in {folder} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def storage_dtype(stored: str, kind: str, run_dtype: torch.dtype) -> torch.dtype:
    """The type a tensor is kept in on the device."""
    if kind == "int":
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in ("F32", "F64"):
        return torch.float32
    return torch.bfloat16


def check_against(folder: str, declared: Mapping[str, ParamDecl],
                  found: Mapping[str, Tuple[str, Tuple[int, ...]]]) -> None:
    """Raise one WeightError listing every disagreement between ``declared`` and ``found``."""
    missing = [n for n in declared if n not in found]
    unexpected = [n for n in found if n not in declared
                  and not any(fnmatch.fnmatch(n, pat) for pat in IGNORED_TENSORS)]
    wrong = []
    for n, decl in declared.items():
        if n not in found:
            continue
        stored, shape = found[n]
        if tuple(shape) != tuple(decl.shape):
            wrong.append(f"{n}: expected {list(decl.shape)}, found {list(shape)}")
        elif decl.kind == "float" and stored not in _FLOATS:
            wrong.append(f"{n}: expected a floating type, found {stored}")
        elif decl.kind == "int" and stored not in _INTS:
            wrong.append(f"{n}: expected an integer type, found {stored}")
    if missing or unexpected or wrong:
        raise WeightError(folder, sorted(missing), sorted(unexpected), wrong)


def load_tensors(folder: str, declared: Mapping[str, ParamDecl], run_dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    """Read, check and move to ``device`` every declared tensor of ``folder``."""
    files, where = open_model_files(folder)
    found = {name: files[fname].info(name) for name, fname in where.items()}
    check_against(folder, declared, found)
    out: Dict[str, torch.Tensor] = {}
    for name, decl in declared.items():
        stored, _ = found[name]
        src = files[where[name]].tensor(name)
        target = storage_dtype(stored, decl.kind, run_dtype)
        if src.dtype == target:
            out[name] = src.to(device)                 # one copy: mapped file -> device
        else:
            out[name] = src.to(device).to(target)      # widen or narrow on the device
    for f in files.values():
        f.close()
    return out
