"""Scratch memory of a step: named device buffers that are kept and reused.

Layers run one after another and ask for the same names, so a step's scratch is
as large as its largest layer needs.  A buffer grows when a larger request
comes, and growing moves it: ``moves`` counts how often that has happened, so
that whoever recorded addresses of this workspace (captured CUDA graphs) can tell
that they are stale.  The captured decode steps of all batch sizes share one
workspace of their own, apart from the one of prompt steps, whose growth would
otherwise move what they point to.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._flat: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._last: Dict[Tuple[str, torch.dtype], Tuple[tuple, torch.Tensor]] = {}   # the view handed out last
        self.moves = 0

    def buf(self, name: str, shape, dtype: torch.dtype, zeros: bool = False) -> torch.Tensor:
        """The named buffer, at least as large as ``shape``.  ``zeros``: the memory is zero when it is first
        handed out (and when it has grown); afterwards it holds what its users left."""
        key = (name, dtype)
        shape = tuple(shape)
        last = self._last.get(key)
        if last is not None and last[0] == shape:
            return last[1]                      # steps of one shape ask for the same views again and again
        n = 1
        for s in shape:
            n *= int(s)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < n:
            if flat is not None:
                self.moves += 1                 # a buffer someone may point to is replaced
            make = torch.zeros if zeros else torch.empty
            flat = make(max(n, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
        view = flat[:n].view(*shape)
        self._last[key] = (shape, view)
        return view

    def zero(self, name: str) -> None:
        """Set every buffer of this name to zero (whatever its element type)."""
        for (n, _), flat in self._flat.items():
            if n == name:
                flat.zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())
