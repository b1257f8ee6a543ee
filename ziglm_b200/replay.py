"""Trace replay: drives the engine's own step function with given token ids and writes logits.

There is no forward pass, cache or loader here: requests are mapped to slots of
the engine, each line of the trace becomes one call of ``Engine.step``, and the
logits it returns are written out.  The reference has no such program; its
closest calls are the public ``prefill``/``decode`` (src/engine.zig:321-348).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List, Optional

from .cache import PAGE_SIZE
from .engine import Engine, EngineOptions


def _parse(argv: Optional[List[str]]) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                   help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    p.add_argument("--out", required=True, help="folder the logits are written to")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time, each request rounded up to a multiple of 64")
    return p.parse_args(argv)


def main(argv: Optional[List[str]] = None, stdin=None, stdout=None) -> int:
    args = _parse(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    os.makedirs(args.out, exist_ok=True)
    max_tokens = max(PAGE_SIZE, -(-args.max_tokens // PAGE_SIZE) * PAGE_SIZE)
    # a request may be as long as the cache: a trace is a check of arithmetic, and the rotation of a position is
    # defined beyond the positions config.json says the model was trained on
    options = EngineOptions(dtype=args.dtype, max_tokens=max_tokens, max_batch=max_tokens // PAGE_SIZE,
                            max_seq_len=max_tokens, beyond_max_positions=True)
    engine = Engine.load(args.model, options)
    slot_of: Dict[str, int] = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_no = rec["step"]
        entries = []
        want = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slot_of:
                slot_of[rid] = engine.alloc_slot()
            entries.append((slot_of[rid], [int(t) for t in e["tokens"]]))
            want.append([int(i) for i in e.get("want", [])])
        if entries:
            logits = engine.step(entries, want)
            if logits is not None:
                data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step_no}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step_no}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slot_of:
                engine.free_slot(slot_of.pop(rid))
        print(f"done {step_no}", file=stdout, flush=True)
    return 0
