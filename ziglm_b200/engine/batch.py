"""A step's batch: the tokens it brings, where they sit, and what is wanted back.

The host lists of a step (per sequence: slot, past length, new tokens, wanted
places) are packed into one int32 buffer in pinned memory and copied to the
device in one transfer; the kernels read everything that varies from step to step
from there (the reference does the same for its single sequence with an 8-byte
{token, pos} block so that its decode graph can be replayed,
src/cuda_model.zig:1017-1048).

Token t of the packed stream belongs to sequence ``seq_of_token[t]`` of the batch
and sits at position ``positions[t]`` of that sequence; sequence b owns tokens
``cu_seqlens[b] .. cu_seqlens[b+1]``.  Block tables are per cache group, one row
per sequence of the batch in batch order.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


def _align(n: int, a: int = 4) -> int:
    return -(-n // a) * a


@dataclass
class BatchLayout:
    """Offsets (in int32 elements) of the sections of the packed buffer."""
    n_tokens: int
    n_seqs: int
    n_want: int
    table_widths: Tuple[int, ...]
    offsets: Dict[str, int] = field(default_factory=dict)
    total: int = 0

    def __post_init__(self) -> None:
        off = 0
        for name, n in (("tokens", self.n_tokens), ("positions", self.n_tokens), ("seq_of_token", self.n_tokens),
                        ("cu_seqlens", self.n_seqs + 1), ("past_lens", self.n_seqs), ("total_lens", self.n_seqs),
                        ("slots", self.n_seqs), ("want_rows", self.n_want)):
            self.offsets[name] = off
            off += _align(n)
        for g, w in enumerate(self.table_widths):
            self.offsets[f"table{g}"] = off
            off += _align(self.n_seqs * w)
        self.total = max(off, 4)


@dataclass
class StepContext:
    """Everything a part may read about the running step."""
    n_tokens: int
    n_seqs: int
    n_want: int
    tokens: torch.Tensor            # int32 [T]
    positions: torch.Tensor         # int32 [T]
    seq_of_token: torch.Tensor      # int32 [T]
    cu_seqlens: torch.Tensor        # int32 [B+1]
    past_lens: torch.Tensor         # int32 [B] length of each sequence before the step
    total_lens: torch.Tensor        # int32 [B] and after it
    slots: torch.Tensor             # int32 [B] slot of each sequence (indexes per-sequence state)
    want_rows: torch.Tensor         # int32 [W] rows of the packed stream whose logits are wanted
    block_tables: List[torch.Tensor]    # per cache group: int32 [B, width]
    single_token: bool              # every sequence brings exactly one token
    max_new: int                    # most tokens one sequence brings (host value)
    max_total: int                  # longest sequence after the step (host value)
    dtype: torch.dtype
    device: torch.device
    ws: Any                         # Workspace
    io: List[Any] = field(default_factory=list)     # LayerIO per place of the schedule
    host_past_lens: List[int] = field(default_factory=list)
    host_new_lens: List[int] = field(default_factory=list)
    host_slots: List[int] = field(default_factory=list)


def pack_batch(layout: BatchLayout, host: torch.Tensor, slots: Sequence[int], past_lens: Sequence[int],
               new_tokens: Sequence[Sequence[int]], want_rows: Sequence[int], tables: Sequence[Any]) -> None:
    """Fill the pinned int32 buffer ``host`` according to ``layout``.  ``tables``: per cache group the block
    table rows of the batch's sequences, a list of lists or an int32 array [B, width]."""
    o = layout.offsets
    buf = host.numpy()                       # shares the pinned memory
    B = len(slots)

    def put(name: str, values) -> None:
        n = len(values)
        if n:
            buf[o[name]:o[name] + n] = values

    if all(len(t) == 1 for t in new_tokens):
        # a decode step: one token per sequence, position = length so far
        put("tokens", [t[0] for t in new_tokens])
        put("positions", past_lens)
        put("seq_of_token", _ARANGE[:B] if B <= len(_ARANGE) else np.arange(B, dtype=np.int32))
        put("cu_seqlens", _ARANGE[:B + 1] if B < len(_ARANGE) else np.arange(B + 1, dtype=np.int32))
        put("past_lens", past_lens)
        put("total_lens", [p + 1 for p in past_lens])
    else:
        toks: List[int] = []
        pos: List[int] = []
        seq: List[int] = []
        cu = [0]
        for b, (past, new) in enumerate(zip(past_lens, new_tokens)):
            toks.extend(new)
            pos.extend(range(past, past + len(new)))
            seq.extend([b] * len(new))
            cu.append(cu[-1] + len(new))
        put("tokens", toks); put("positions", pos); put("seq_of_token", seq); put("cu_seqlens", cu)
        put("past_lens", past_lens)
        put("total_lens", [p + len(n) for p, n in zip(past_lens, new_tokens)])
    put("slots", slots)
    put("want_rows", want_rows)
    for g, rows in enumerate(tables):
        flat = np.asarray(rows, dtype=np.int32).reshape(-1)
        put(f"table{g}", flat)


_ARANGE = np.arange(4097, dtype=np.int32)


def views(layout: BatchLayout, dev: torch.Tensor) -> Dict[str, Any]:
    """Device views of the sections of a packed buffer."""
    o = layout.offsets
    T, B, W = layout.n_tokens, layout.n_seqs, layout.n_want

    def sec(name: str, n: int) -> torch.Tensor:
        return dev[o[name]:o[name] + n]

    out: Dict[str, Any] = {
        "tokens": sec("tokens", T), "positions": sec("positions", T), "seq_of_token": sec("seq_of_token", T),
        "cu_seqlens": sec("cu_seqlens", B + 1), "past_lens": sec("past_lens", B), "total_lens": sec("total_lens", B),
        "slots": sec("slots", B), "want_rows": sec("want_rows", W),
    }
    out["block_tables"] = [sec(f"table{g}", B * w).view(B, w) for g, w in enumerate(layout.table_widths)]
    return out
