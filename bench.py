#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
    python bench.py --case prefill|decode [--layers L] [--batch B] [--context C]    one phase alone, for profilers
    python bench.py --case reference-kernels [--context C]     the reference's CUDA kernels alone, if they were built

A "step" is one decode step of a batch of 8 sequences at a context of 4096
tokens.  ``value`` is decoded tokens a second, timed on the device with CUDA
events over exactly K steps after W warm-up steps; ``e2e`` is the same loop
through the Python entry point with host token ids in (pinned memory, copied to
the device every step) and sampled ids out (read back every step).  The line
also carries the prefill of 2,048 tokens, the decode step's memory roofline,
decode at batch 1 and 64, the SM clocks seen during the timed region and the
number of kernels launched in it.  Weights are random N(0, 0.02) in bfloat16
and token ids are uniform random: there is no dataset or checkpoint here.

The reference (a Zig program with one CUDA file) has no Python package and no
Zig toolchain is installed, so ``--impl reference`` reports itself unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "attention_bias": False,
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
        return out
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(int(float(s[0])))
                mx = max(mx, int(float(s[1])))
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


def decode_bytes(cfg, n_layers, batch, context, bytes_per_el=2):
    """Bytes a decode step has to read: every weight it uses once and the cache of the live requests."""
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * q + 2 * d * kv + q * d + 3 * d * i + 2 * d
    weights = n_layers * per_layer + v * d + d                 # the head; the embedding is read for `batch` rows only
    cache = n_layers * 2 * kv * context * batch
    return (weights + cache) * bytes_per_el + batch * d * bytes_per_el


def prefill_flops(cfg, n_layers, tokens):
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2 * tokens * (d * q + 2 * d * kv + q * d + 3 * d * i)
    attn = 2 * 2 * q * tokens * (tokens + 1) / 2               # QK^T and PV over the causal half
    return n_layers * (linear + attn) + 2 * d * v              # the head runs on the last token only


def run_ours(args):
    import torch
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams, config_from_dict, kernels
    from ziglm_b200.sampling.device import DeviceSampler

    torch.cuda.set_device(0)
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg["num_hidden_layers"] = n_layers
    pk = peaks()
    steps, warmup = args.steps, max(3, args.warmup)
    slack = 64
    max_seq = CONTEXT + slack

    def make_engine(batch):
        opts = EngineOptions(dtype="bfloat16", max_batch=batch, max_seq_len=max_seq,
                             max_tokens=batch * (-(-max_seq // 64) * 64), seed=1234)
        return Engine.from_config(config_from_dict(cfg), opts)

    gen = torch.Generator().manual_seed(7)

    def random_ids(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()

    def fill(engine, batch, context):
        """Give `batch` sequences `context` cached tokens each, by real prompt steps of at most 2048 tokens."""
        slots = [engine.alloc_slot() for _ in range(batch)]
        for s in slots:
            done = 0
            while done < context:
                n = min(2048, context - done)
                engine.step([(s, random_ids(n))], [[]])
                done += n
        return slots

    def time_decode(engine, slots, n_warm, n_steps, flush=None):
        """Device time of n_steps decode steps (ms per step) and the kernels launched in them."""
        ids = [random_ids(len(slots)) for _ in range(n_warm + n_steps)]
        for k in range(n_warm):
            engine.step([(s, [t]) for s, t in zip(slots, ids[k])])
        torch.cuda.synchronize()
        kernels.reset_launches()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(n_warm, n_warm + n_steps):
            engine.step([(s, [t]) for s, t in zip(slots, ids[k])])
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / n_steps, kernels.launches() + engine.graph_launched_kernels()

    result = {}
    # ---------------------------------------------------------------- prefill, 2048 tokens of one sequence
    engine = make_engine(8)
    prompt = random_ids(PREFILL_TOKENS)
    times = []
    for k in range(3 + 3):
        slot = engine.alloc_slot()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([(slot, prompt)])
        e.record()
        torch.cuda.synchronize()
        if k >= 3:
            times.append(s.elapsed_time(e))
        engine.free_slot(slot)
    pre_ms = sorted(times)[len(times) // 2]
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    result["prefill"] = {"value": round(PREFILL_TOKENS / pre_ms * 1000.0, 1), "tokens": PREFILL_TOKENS,
                         "ms": round(pre_ms, 3),
                         "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---------------------------------------------------------------- decode, batch 8 at the context length
    batch = 8
    start_ctx = CONTEXT - (warmup + steps) - 1
    slots = fill(engine, batch, max(1, start_ctx))
    with ClockSampler() as clocks:
        ms, launched = time_decode(engine, slots, warmup, steps)
    clock_summary = clocks.summary()
    tok_s = batch / ms * 1000.0
    bytes_step = decode_bytes(cfg, n_layers, batch, CONTEXT)
    achieved = bytes_step / (ms * 1e-3) / 1e9

    # ---------------------------------------------------------------- the same through the Python entry point
    sampler = DeviceSampler(engine)
    params = SamplerParams(greedy=True)
    pinned = torch.empty(batch, dtype=torch.int32).pin_memory()
    for s in slots:
        engine.free_slot(s)
    slots = fill(engine, batch, max(1, start_ctx))
    tokens = random_ids(batch)
    e2e_steps = steps
    for k in range(warmup):
        tokens = sampler.step_and_sample([(s, [t]) for s, t in zip(slots, tokens)], list(range(batch)),
                                         [[]] * batch, [k] * batch, params)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for k in range(e2e_steps):
        tokens = sampler.step_and_sample([(s, [t]) for s, t in zip(slots, tokens)], list(range(batch)),
                                         [[]] * batch, [k] * batch, params)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000.0 / e2e_steps
    h2d = engine.last_step_h2d_bytes
    for s in slots:
        engine.free_slot(s)
    del sampler

    # ---------------------------------------------------------------- decode at batch 1 and 64
    points = {}
    s1 = fill(engine, 1, max(1, start_ctx))
    ms1, _ = time_decode(engine, s1, warmup, steps)
    points["decode_b1"] = round(1 / ms1 * 1000.0, 1)
    engine.free_slot(s1[0])
    del engine
    torch.cuda.empty_cache()
    engine = make_engine(64)
    s64 = fill(engine, 64, max(1, start_ctx))
    ms64, _ = time_decode(engine, s64, warmup, steps)
    points["decode_b64"] = round(64 / ms64 * 1000.0, 1)
    points["decode_b1_hbm_frac"] = round(decode_bytes(cfg, n_layers, 1, CONTEXT) / (ms1 * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    points["decode_b64_hbm_frac"] = round(decode_bytes(cfg, n_layers, 64, CONTEXT) / (ms64 * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    line = {
        "metric": "decode tok/s at batch 8 (Llama-3.1-8B shape, context 4096)",
        "value": round(tok_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Llama-3.1-8B shape", "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": n_layers, "layers_of_config": full_layers, "hidden_size": cfg["hidden_size"],
            "intermediate_size": cfg["intermediate_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"],
            "rope_theta": cfg["rope_theta"], "rope_scaling": "llama3 factor 8 low 1 high 4 orig 8192",
            "rms_norm_eps": cfg["rms_norm_eps"], "tied": False, "prefill_tokens": PREFILL_TOKENS,
            "l2": "inputs larger than L2 (weights read each step exceed 126 MB)", "peaks": pk["source"],
        },
        "e2e": {"value": round(batch / e2e_ms * 1000.0, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": batch * 4},
        "gpu_launches": int(launched),
        "prefill": result["prefill"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


def run_case(args):
    """A single phase on a (possibly shallower) model, for profilers: the prompt of 2,048 tokens, or decode steps."""
    import torch
    from ziglm_b200 import Engine, EngineOptions, config_from_dict, kernels
    torch.cuda.set_device(0)
    cfg = dict(LLAMA_8B)
    cfg["num_hidden_layers"] = args.layers or cfg["num_hidden_layers"]
    batch, context = args.batch, args.context
    max_seq = max(context, args.prompt_tokens) + 64
    eng = Engine.from_config(config_from_dict(cfg), EngineOptions(
        dtype="bfloat16", max_batch=batch, max_seq_len=max_seq, max_tokens=batch * (-(-max_seq // 64) * 64), seed=1234))
    gen = torch.Generator().manual_seed(7)
    ids = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()
    times = []
    if args.case == "prefill":
        prompt = ids(args.prompt_tokens)
        for k in range(args.warmup + args.steps):
            slot = eng.alloc_slot()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            eng.step([(slot, prompt)])
            e.record()
            torch.cuda.synchronize()
            if k >= args.warmup:
                times.append(s.elapsed_time(e))
            eng.free_slot(slot)
        tokens = args.prompt_tokens
    else:
        slots = [eng.alloc_slot() for _ in range(batch)]
        # the cache is given its length without being computed: a decode step's time does not depend on its content
        grow = {s: context - args.warmup - args.steps - 1 for s in slots}
        eng.cache.slots.reserve(grow)
        eng.cache.slots.advance(grow)
        for k in range(args.warmup + args.steps):
            toks = ids(batch)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            eng.step([(sl, [t]) for sl, t in zip(slots, toks)])
            e.record()
            torch.cuda.synchronize()
            if k >= args.warmup:
                times.append(s.elapsed_time(e))
        tokens = batch
    ms = sorted(times)[len(times) // 2]
    print(json.dumps({"case": args.case, "layers": cfg["num_hidden_layers"], "batch": batch, "context": context,
                      "ms": round(ms, 4), "tok_s": round(tokens / ms * 1000.0, 1),
                      "wait_errors": [kernels.gemm_tc_status(), kernels.attention_tc_status(),
                                      kernels.attention_fmha_status()]}))
    return 0


REFERENCE_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "libziglm_cuda.so")


def run_reference_kernels(args):
    """The reference's own CUDA kernels (its src/cuda_bridge.cu, unmodified, compiled for sm_100a into
    baseline/_ref/libziglm_cuda.so), timed at the shapes of this benchmark and put together in the order its
    decode step calls them for one Llama layer (src/model.zig:600-760): one sequence, float32 activations and
    cache, bf16 weights.  This is not the reference arm (its engine is a Zig program): it says what the
    reference's kernels alone would give on this GPU."""
    import ctypes
    from ctypes import c_float, c_int, c_void_p
    import torch
    if not os.path.isfile(REFERENCE_LIB):
        print(json.dumps({"case": "reference-kernels", "unavailable":
                          "baseline/_ref/libziglm_cuda.so is not there (build it from the reference's "
                          "src/cuda_bridge.cu with nvcc -shared -gencode arch=compute_100a,code=sm_100a)"}))
        return 0
    lib = ctypes.CDLL(REFERENCE_LIB)
    P = c_void_p
    protos = {
        "cuda_gemv_bf16": [P, P, P, c_int, c_int, P],
        "cuda_rmsnorm": [P, P, P, c_int, c_float, c_int, P],
        "cuda_rope": [P, P, c_int, c_int, c_int, c_int, c_int, c_float, P],
        "cuda_kv_cache_put": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, P],
        "cuda_attention_forward": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, P],
        "cuda_swiglu": [P, P, P, c_int, P],
        "cuda_add": [P, P, c_int, P],
    }
    for name, argtypes in protos.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, None
    torch.cuda.set_device(0)
    dev = "cuda:0"
    c = LLAMA_8B
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    ctx = args.context
    stream = torch.cuda.current_stream().cuda_stream
    bf = lambda r, k: (torch.randn(r, k, device=dev) * 0.02).to(torch.bfloat16)
    f32 = lambda n: torch.randn(n, device=dev)
    w = {"q": bf(nh * hd, H), "k": bf(nkv * hd, H), "v": bf(nkv * hd, H), "o": bf(H, nh * hd), "gate": bf(I, H),
         "up": bf(I, H), "down": bf(H, I), "head": bf(V, H)}
    g1, g2 = torch.ones(H, device=dev), torch.ones(H, device=dev)
    x, h, q, k, v, att, o = f32(H), f32(H), f32(nh * hd), f32(nkv * hd), f32(nkv * hd), f32(nh * hd), f32(H)
    gate, up, act, down, logits = f32(I), f32(I), f32(I), f32(H), f32(V)
    kc = torch.randn(ctx, nkv * hd, device=dev)
    vc = torch.randn(ctx, nkv * hd, device=dev)
    pos, eps, scale = ctx - 1, c["rms_norm_eps"], 1.0 / hd ** 0.5
    p = lambda t: t.data_ptr()
    steps = {
        "rmsnorm": lambda: lib.cuda_rmsnorm(p(x), p(g1), p(h), H, eps, 0, stream),
        "gemv_q": lambda: lib.cuda_gemv_bf16(p(w["q"]), p(h), p(q), nh * hd, H, stream),
        "gemv_k": lambda: lib.cuda_gemv_bf16(p(w["k"]), p(h), p(k), nkv * hd, H, stream),
        "gemv_v": lambda: lib.cuda_gemv_bf16(p(w["v"]), p(h), p(v), nkv * hd, H, stream),
        "rope": lambda: lib.cuda_rope(p(q), p(k), pos, nh, nkv, hd, hd, c["rope_theta"], stream),
        "kv_put": lambda: lib.cuda_kv_cache_put(p(kc), p(vc), p(k), p(v), 0, pos, ctx, nkv, hd, nkv * hd, stream),
        "attention": lambda: lib.cuda_attention_forward(p(q), p(kc), p(vc), p(att), 0, pos, ctx, nh, nkv, hd, nkv * hd,
                                                        scale, 0.0, 0, stream),
        "gemv_o": lambda: lib.cuda_gemv_bf16(p(w["o"]), p(att), p(o), H, nh * hd, stream),
        "add_1": lambda: lib.cuda_add(p(x), p(o), H, stream),
        "rmsnorm_2": lambda: lib.cuda_rmsnorm(p(x), p(g2), p(h), H, eps, 0, stream),
        "gemv_gate": lambda: lib.cuda_gemv_bf16(p(w["gate"]), p(h), p(gate), I, H, stream),
        "gemv_up": lambda: lib.cuda_gemv_bf16(p(w["up"]), p(h), p(up), I, H, stream),
        "swiglu": lambda: lib.cuda_swiglu(p(gate), p(up), p(act), I, stream),
        "gemv_down": lambda: lib.cuda_gemv_bf16(p(w["down"]), p(act), p(down), H, I, stream),
        "add_2": lambda: lib.cuda_add(p(x), p(down), H, stream),
    }
    # The reference's cuda_argmax is left out: it hands its kernels the host-side names of two __device__
    # arrays as pointers (src/cuda_bridge.cu:2943-2944, 3075-3076), which is an illegal memory access on
    # this GPU; it ran here once and is not run again.
    tail = {
        "gemv_head": lambda: lib.cuda_gemv_bf16(p(w["head"]), p(h), p(logits), V, H, stream),
    }
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)       # larger than L2

    def timed(fn, reps):
        ts = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1000.0)
        return sorted(ts)[len(ts) // 2]

    for name, fn in {**steps, **tail}.items():        # one by one first: a failing launch is named
        fn()
        try:
            torch.cuda.synchronize()
        except RuntimeError as e:
            print(json.dumps({"case": "reference-kernels", "unavailable": "%s failed: %s" % (name, str(e).splitlines()[0])}))
            return 0
    each = {name: round(timed(fn, 7), 1) for name, fn in {**steps, **tail}.items()}

    def layer():
        for fn in steps.values():
            fn()
    layer_us = timed(layer, 7)
    tail_us = each["rmsnorm"] + each["gemv_head"]
    token_ms = (layer_us * c["num_hidden_layers"] + tail_us) / 1000.0
    print(json.dumps({"case": "reference-kernels", "what": "simonproyt/ziglm src/cuda_bridge.cu compiled for sm_100a, one "
                      "sequence, context %d, Llama-3.1-8B layer shapes; L2 flushed before every timing; without its argmax "
                      "(faults here)" % ctx,
                      "kernel_us": each, "layer_us": round(layer_us, 1),
                      "decode_b1_ms_per_token": round(token_ms, 3), "decode_b1_tok_s": round(1000.0 / token_ms, 1)}))
    return 0


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--case", default="full", choices=["full", "prefill", "decode", "reference-kernels"],
                    help="full: the whole measurement; prefill / decode: that phase alone (for profilers); "
                         "reference-kernels: the reference's CUDA kernels alone, if they were built")
    ap.add_argument("--batch", type=int, default=8, help="--case decode: sequences in the batch")
    ap.add_argument("--context", type=int, default=CONTEXT, help="--case decode: tokens each sequence holds")
    ap.add_argument("--prompt-tokens", type=int, default=PREFILL_TOKENS, help="--case prefill: tokens of the prompt")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Zig program (no setup.py or pyproject.toml, pip reports it is not "
                          "installable) and no Zig toolchain is installed here or on the GPU box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    if args.case == "reference-kernels":
        return run_reference_kernels(args)
    if args.case != "full":
        return run_case(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
