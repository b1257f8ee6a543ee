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
    """The roofline's bytes and FLOPs, checked against sources that are not bench.py's formulas: the tensors
    the model declares (what a decode step has to read), the figures the published shapes are known by, and a
    count made tensor by tensor."""
    sys.path.insert(0, ROOT)
    import bench
    from ziglm_b200 import config_from_dict
    from ziglm_b200.engine.model import declare_parameters
    for name, cfg, batch, context in (("8b", bench.LLAMA_8B, 8, 4096), ("1b", bench.LLAMA_1B, 64, 600),
                                      ("13b", bench.LLAMA_13B, 8, 2304)):
        conf = config_from_dict(cfg)
        declared = declare_parameters(conf.model_spec())
        elements = {n: 1 for n in declared}
        for n, decl in declared.items():
            for k in decl.shape:
                elements[n] *= k
        # every declared tensor is read once, except the embedding table of a model with a head of its own,
        # of which the step gathers `batch` rows; the cache: keys and values of every layer for every live token
        weights = sum(elements.values())
        if not conf.tie_word_embeddings:
            weights -= elements["model.embed_tokens.weight"]
        kv_per_token = 2 * conf.num_hidden_layers * conf.num_key_value_heads * conf.head_dim
        want = 2 * (weights + kv_per_token * batch * context + batch * conf.hidden_size)
        got = bench.decode_bytes(cfg, conf.num_hidden_layers, batch, context)
        assert abs(got - want) <= 1e-9 * want, name
        assert bench.decode_bytes(cfg, conf.num_hidden_layers, batch, 0, cached_tokens=batch * context) == got
    # the figures the shapes are known by: 8.03 B parameters (15.01 GB of them read by a step), 128 KiB of cache a token
    assert abs(bench.decode_bytes(bench.LLAMA_8B, 32, 1, 0) - 15.01e9) < 0.01e9
    assert bench.decode_bytes(bench.LLAMA_8B, 32, 1, 1) - bench.decode_bytes(bench.LLAMA_8B, 32, 1, 0) == 128 * 1024
    assert abs(bench.decode_bytes(bench.LLAMA_8B, 32, 8, 4096) - 19.30e9) < 0.01e9
    # the prompt, product by product: 2 FLOPs per weight element and token, the causal half of attention
    # (scores and weighted values, 2 FLOPs each per query, key and head dimension), the head for one row
    cfg = bench.LLAMA_8B
    T, flops = 2048, 0
    for n, decl in declare_parameters(config_from_dict(cfg).model_spec()).items():
        if len(decl.shape) == 2 and "layers." in n:
            flops += 2 * T * decl.shape[0] * decl.shape[1]
    flops += 32 * 2 * 2 * (32 * 128) * sum(p + 1 for p in range(T))
    flops += 2 * 4096 * 128256
    assert abs(bench.prefill_flops(cfg, 32, T) - flops) <= 1e-9 * flops
    assert abs(flops - 29.69e12) < 0.01e12


import pytest


@pytest.mark.gpu
def test_the_line_of_a_shallow_run_has_every_key_of_the_contract():
    """`bench.py` on two layers of the benchmarked shape: one JSON line with the metric, the end-to-end figure and
    its bytes, the prefill and roofline records, the points, the clocks, a launch count that is the kernels of the
    timed steps, and a flat `config` of at most 20 keys that names both layer counts."""
    r = run("--layers", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "prefill", "roofline", "points",
                "clocks", "wait_errors"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 4 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert abs(d["value"] - 8 / d["ms_per_step"] * 1e3) < 1e-2 * d["value"]
    cfg = d["config"]
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    assert cfg["layers"] == 2 and cfg["layers_of_config"] == 32 and cfg["global_batch"] == 8 and cfg["seq_len"] == 4096
    assert set(d["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] == 8 * 4
    assert 0 < d["e2e"]["value"] <= 1.05 * d["value"]
    assert set(d["prefill"]) >= {"value", "tokens", "ms", "frac"} and d["prefill"]["tokens"] == 2048
    assert set(d["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac"} and d["roofline"]["bound"] == "hbm"
    assert abs(d["roofline"]["frac"] - d["roofline"]["achieved"] / d["roofline"]["peak"]) < 1e-3
    assert {"decode_b1", "decode_b64"} <= set(d["points"])
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    # a decode step of two layers at these widths: embedding, first norm, five launches a layer, last norm, head,
    # the greedy choice
    assert d["gpu_launches"] == 4 * (5 * 2 + 5)
    assert d["wait_errors"] == [0, 0, 0]
