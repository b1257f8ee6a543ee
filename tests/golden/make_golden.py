"""Writes tests/golden/plain_tiny.json: a few logits of the plain implementation on the tiny configurations.

The reference's own model code is Zig and cannot be compiled or imported in this
environment, so these outputs come from tests/plain_llama.py (written from the
reference's formulas) and pin it against accidental change; they are not outputs
of the reference.  The parts of the plain implementation are checked against the
reference's own CUDA kernels separately (make_reference_kernel_golden.py).

    python tests/golden/make_golden.py
"""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import torch  # noqa: E402

import helpers  # noqa: E402

out = {}
for name, seed in (("A", 101), ("B", 202), ("F", 303), ("G", 404)):
    cfg = helpers.CONFIGS[name]
    tokens = helpers.random_tokens(9, cfg["vocab_size"], seed)
    with tempfile.TemporaryDirectory() as tmp:
        folder = helpers.make_folder(tmp, cfg, seed, torch.float32, helpers.NORM_JITTER[name])
        logits = helpers.plain_logits(folder, tokens)
    out[name] = {"seed": seed, "tokens": tokens, "last_logits_head": [round(v, 8) for v in logits[-1, :8].tolist()],
                 "abs_sum": logits.abs().sum().item()}
json.dump(out, open(os.path.join(HERE, "plain_tiny.json"), "w"), indent=1)
print(json.dumps(out, indent=1))
