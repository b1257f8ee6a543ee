"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2; the
reference arm says in one JSON line why it cannot run and exits 0; the byte and FLOP counts that the roofline
fractions rest on are what the shapes give."""
import json
import os
import subprocess
import sys

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
BENCH = os.path.join(ROOT, "bench.py")


def run(*args):
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=300, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    r = run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_prints_its_unavailable_line():
    r = run("--impl", "reference", "--gpus", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_byte_and_flop_counts():
    sys.path.insert(0, ROOT)
    import bench
    cfg = bench.LLAMA_8B
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * q + 2 * d * kv + q * d + 3 * d * i
    # a decode step reads every weight it uses once (the embedding rows it gathers are not counted) and the
    # keys and values of the live requests
    want = 2 * (32 * per_layer + d * v) + 8 * 4096 * 32 * 2 * kv * 2
    got = bench.decode_bytes(cfg, 32, 8, 4096)
    assert abs(got - want) <= 0.01 * want
    # the prompt: products of every token, the causal half of attention, the head for one row
    flops = bench.prefill_flops(cfg, 32, 2048)
    want_f = 32 * (2 * 2048 * per_layer + 2 * 2 * q * 2048 * 2049 / 2) + 2 * d * v
    assert abs(flops - want_f) <= 1e-6 * want_f
