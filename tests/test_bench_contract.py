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
