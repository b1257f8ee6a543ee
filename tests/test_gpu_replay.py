"""bin/trace_run as a user runs it: a process fed JSON lines that answers ``done <step>`` and writes logits.
The same requests are replayed whole, with their last 32 tokens one by one, and in batches of unequal lengths
whose shorter requests end earlier (batch after batch, so that slots and pages are used again), in float32 and
in bfloat16, and every logit row is compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": [5, 11, 17, 70, 45], "B": [1, 9, 23, 40, 97], "H": [7, 128, 50, 100, 66]}


class Replay:
    def __init__(self, folder, dtype, out, max_tokens):
        self.out = out
        self.proc = subprocess.Popen(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step_no = 0

    def step(self, entries, end=()):
        rec = {"step": self.step_no, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.step_no}", f"trace_run answered {line!r}"
        path = os.path.join(self.out, f"{self.step_no}.f32")
        n_want = sum(len(e["want"]) for e in entries)
        self.step_no += 1
        if n_want == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        return torch.from_numpy(data.reshape(n_want, -1).copy())

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=120) == 0


@pytest.mark.parametrize("name", ["A", "B", "H"])          # H: a sliding window of 48 in every layer
@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_replay_schedules(tmp_path, name, dn):
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn]
    cfg = helpers.CONFIGS[name]
    folder = helpers.make_folder(tmp_path, cfg, 31, dtype, helpers.NORM_JITTER[name])
    reqs = [helpers.random_tokens(n, cfg["vocab_size"], 200 + i) for i, n in enumerate(LENGTHS[name])]
    act = None if dn == "float32" else torch.bfloat16
    want = [helpers.plain_logits(folder, r, act=act) for r in reqs]
    # the batched schedule holds at most three requests of at most 128 positions
    rp = Replay(folder, dn, str(tmp_path / "logits"), max_tokens=3 * 128)
    try:
        # 1. each request alone and whole
        for i, r in enumerate(reqs):
            got = rp.step([{"id": f"w{i}", "tokens": r, "want": list(range(len(r)))}], end=[f"w{i}"])
            helpers.assert_close(got, want[i], dtype, f"{name} {dn} whole, request {i}")
        # 2. the last 32 tokens one by one; nothing is wanted from the first part of requests 0 and 3
        for i, r in enumerate(reqs):
            head = max(1, len(r) - 32)
            w = [] if i in (0, 3) else list(range(head))
            got = rp.step([{"id": f"t{i}", "tokens": r[:head], "want": w}])
            if w:
                helpers.assert_close(got, want[i][:head], dtype, f"{name} {dn} tail, head of request {i}")
            for p in range(head, len(r)):
                got = rp.step([{"id": f"t{i}", "tokens": [r[p]], "want": [0]}], end=[f"t{i}"] if p == len(r) - 1 else [])
                helpers.assert_close(got, want[i][p:p + 1], dtype, f"{name} {dn} tail, request {i} position {p}")
            if head == len(r):
                rp.step([], end=[f"t{i}"])
        # 3. batches of unequal lengths, batch after batch
        order = sorted(range(len(reqs)), key=lambda i: len(reqs[i]))
        for batch in ([order[0], order[4], order[2]], [order[3], order[1]]):
            used = {i: 0 for i in batch}
            live = list(batch)
            first = True
            while live:
                entries = []
                for i in live:
                    n = max(1, len(reqs[i]) - 7 * (i + 1)) if first else 1
                    n = min(n, len(reqs[i]) - used[i])
                    entries.append({"id": f"b{i}", "tokens": reqs[i][used[i]:used[i] + n], "want": list(range(n))})
                ending = [f"b{i}" for i, e in zip(live, entries) if used[i] + len(e["tokens"]) == len(reqs[i])]
                got = rp.step(entries, end=ending)
                at = 0
                for i, e in zip(list(live), entries):
                    n = len(e["tokens"])
                    helpers.assert_close(got[at:at + n], want[i][used[i]:used[i] + n], dtype,
                                         f"{name} {dn} batched, request {i} from {used[i]}")
                    at += n
                    used[i] += n
                    if used[i] == len(reqs[i]):
                        live.remove(i)
                first = False
    finally:
        rp.close()


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_replay_runs_positions_beyond_those_the_configuration_names(tmp_path, dn):
    """A trace checks arithmetic: a request may be as long as the cache it was given, although config.json says the
    model knows 64 positions (the rotation of a position is defined for every position; llama3 stretching reads
    its own original length, not this one)."""
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dn]
    cfg = dict(helpers.TINY_B, max_position_embeddings=64)
    folder = helpers.make_folder(tmp_path, cfg, 33, dtype, 0.1)
    r = helpers.random_tokens(150, cfg["vocab_size"], 77)
    want = helpers.plain_logits(folder, r, act=None if dn == "float32" else torch.bfloat16)
    rp = Replay(folder, dn, str(tmp_path / "logits"), max_tokens=192)
    try:
        got = rp.step([{"id": "a", "tokens": r[:140], "want": list(range(140))}])
        helpers.assert_close(got, want[:140], dtype, f"{dn} prompt past position 64")
        for p in range(140, 150):
            got = rp.step([{"id": "a", "tokens": [r[p]], "want": [0]}], end=["a"] if p == 149 else [])
            helpers.assert_close(got, want[p:p + 1], dtype, f"{dn} position {p}")
    finally:
        rp.close()


def test_replay_from_a_fresh_checkout_as_another_user(tmp_path):
    """A copy of the sources without built files, run with an empty HOME: what has to be compiled is compiled at
    the first call, with a line now and then on standard error."""
    import shutil
    fresh = tmp_path / "fresh"
    for part in ("ziglm_b200", "bin"):               # what a checkout holds of the product, without built files
        shutil.copytree(os.path.join(ROOT, part), fresh / part,
                        ignore=shutil.ignore_patterns("_build", "__pycache__", "*.so"))
    folder = helpers.make_folder(tmp_path, helpers.TINY_A, 5, torch.float32)
    home = tmp_path / "home"
    home.mkdir()
    env = {"PATH": os.environ.get("PATH", ""), "HOME": str(home)}
    for k in ("LD_LIBRARY_PATH", "CUDA_HOME", "CUDA_VISIBLE_DEVICES", "VIRTUAL_ENV"):
        if k in os.environ:
            env[k] = os.environ[k]
    toks = helpers.random_tokens(9, 256, 1)
    trace = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [8]}], "end": ["a"]}) + "\n"
    r = subprocess.run([sys.executable, str(fresh / "bin" / "trace_run"), "--model", folder, "--dtype", "float32", "--out",
                        str(tmp_path / "o"), "--max-tokens", "64"], input=trace, capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == "done 0" and "compiling" in r.stderr
    got = torch.from_numpy(np.fromfile(str(tmp_path / "o" / "0.f32"), dtype="<f4").reshape(1, -1).copy())
    helpers.assert_close(got, helpers.plain_logits(folder, toks)[8:9], torch.float32, "fresh checkout")
