"""Generation through the entry points: greedy against the plain implementation, stop tokens, more requests
than slots, sampling against the plain sampler chain, the command line."""
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen")
    out = {}
    for name in ("A", "B"):
        for dn, dtype in DTYPES.items():
            # a larger spread of the weights separates the logits, so that greedy choices do not hinge on rounding
            out[(name, dn)] = helpers.make_folder(tmp, helpers.CONFIGS[name], 23, dtype, helpers.NORM_JITTER[name], std=0.08)
    return out


def plain_greedy(folder, prompt, n, act, stop=()):
    cfg, w = helpers.read_folder(folder)
    seq, out = list(prompt), []
    for _ in range(n):
        tok = P.greedy(P.forward(cfg, w, seq, act=act)[-1])
        if tok in stop:
            break
        out.append(tok); seq.append(tok)
    return out


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_greedy_generation_matches_the_plain_implementation(models, name, dn):
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams
    folder = models[(name, dn)]
    V = helpers.CONFIGS[name]["vocab_size"]
    eng = Engine.load(folder, EngineOptions(dtype=dn, max_tokens=512, max_batch=3))
    prompts = [helpers.random_tokens(n, V, 60 + n) for n in (3, 12, 1, 30, 7)]     # five requests, three slots
    opts = GenerationOptions(max_tokens=10, ignore_eos=True, sampler=SamplerParams(greedy=True))
    results, stats = eng.generate(prompts, opts)
    act = None if dn == "float32" else torch.bfloat16
    for p, r in zip(prompts, results):
        assert r.tokens == plain_greedy(folder, p, 10, act), f"prompt of {len(p)} tokens"
        assert r.finish_reason == "length"
    assert stats.prompt_tokens == sum(len(p) for p in prompts) and stats.completion_tokens == 50
    assert stats.prefill_time_ms > 0 and stats.generation_time_ms > 0
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0
    # one prompt given as a plain list of ids
    single, _ = eng.generate(prompts[1], opts)
    assert single.tokens == results[1].tokens


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_a_model_made_on_the_device_holds_the_tensors_its_folder_would(tmp_path, dn):
    """``Engine.from_config(config, seed)`` fills its weights on the device; ``write_random_model(config, seed)``
    computes them on the host.  Both are the same function of (seed, tensor name, element), so the two engines
    give the same logits bit for bit and the plain implementation can check a model that was never written."""
    from ziglm_b200 import Engine, EngineOptions, config_from_dict, write_random_model
    cfg = helpers.TINY_B
    folder = str(tmp_path / "host_made")
    write_random_model(folder, config_from_dict(cfg), 31, dtype=DTYPES[dn], std=0.05, norm_jitter=0.1,
                       device=torch.device("cpu"))
    opts = EngineOptions(dtype=dn, max_tokens=256, max_batch=2, seed=31)
    made = Engine.from_config(cfg, opts, std=0.05, norm_jitter=0.1)
    loaded = Engine.load(folder, opts)
    _, w = helpers.read_folder(folder)
    assert torch.equal(made.model.embedding.cpu(), w["model.embed_tokens.weight"])
    assert torch.equal(made.model.final_norm.weight.cpu(), w["model.norm.weight"])
    assert torch.equal(made.model.blocks[2].mixer.o.weight.cpu(), w["model.layers.2.self_attn.o_proj.weight"])
    prompt = helpers.random_tokens(21, cfg["vocab_size"], 5)
    a = made.step([(made.alloc_slot(), prompt)], [list(range(21))]).clone()
    b = loaded.step([(loaded.alloc_slot(), prompt)], [list(range(21))]).clone()
    assert torch.equal(a, b)
    helpers.assert_close(a, helpers.plain_logits(folder, prompt, act=None if dn == "float32" else torch.bfloat16),
                         DTYPES[dn], "a model made on the device against the plain model of its folder")


def test_a_wait_that_ran_out_ends_generation_with_a_named_error_and_the_engine_recovers(models):
    """A kernel's bounded wait is made to run out (harmlessly, by the self-test kernel) while an engine lives:
    the engine's check raises an error that names the library and the code, and generation works afterwards."""
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams, kernels
    folder = models[("A", "bfloat16")]
    eng = Engine.load(folder, EngineOptions(dtype="bfloat16", max_tokens=512, max_batch=3))
    opts = GenerationOptions(max_tokens=5, ignore_eos=True, sampler=SamplerParams(greedy=True))
    prompts = [helpers.random_tokens(n, 256, 70 + n) for n in (4, 9)]
    before, _ = eng.generate(prompts, opts)
    eng.check_kernels()                                    # healthy: silent
    assert kernels.wait_selftest("gemm_tc", polls=2048) == (0, 1)
    with pytest.raises(kernels.KernelError, match="gemm_tc: code 90"):
        eng.generate(prompts, opts)                        # found when the first batch ends
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0               # the loop gave every slot back
    after, _ = eng.generate(prompts, opts)
    assert [r.tokens for r in after] == [r.tokens for r in before]


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_running_one_step_ahead_generates_what_the_step_by_step_loop_generates(models, dn, monkeypatch):
    """Generation queues the next step, fed on the device with the ids just sampled, before it reads those ids.
    With the same seed it must give, token for token, what the loop gives that reads every step's ids before it
    launches the next: greedy and sampled (no penalties, which need the ids on the host), with stop tokens that
    end some requests early, more requests than slots, and a request that reaches the end of the context."""
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams
    from ziglm_b200.sampling.device import DeviceSampler
    folder = models[("B", dn)]
    V = helpers.CONFIGS["B"]["vocab_size"]
    eng = Engine.load(folder, EngineOptions(dtype=dn, max_tokens=1024, max_batch=3, max_seq_len=48))
    prompts = [helpers.random_tokens(n, V, 500 + n) for n in (5, 17, 2, 40, 9, 1, 30)]
    launched = []
    real_launch = DeviceSampler.launch
    monkeypatch.setattr(DeviceSampler, "launch", lambda self, *a, **k: (launched.append(k.get("feed") is not None),
                                                                       real_launch(self, *a, **k))[1])
    for sampler in (SamplerParams(greedy=True), SamplerParams(temperature=0.9, top_k=50, top_p=0.95, min_p=0.0, seed=11,
                                                              repetition_penalty=1.0)):
        opts = GenerationOptions(max_tokens=14, sampler=sampler, stop_tokens=[3, 50, 77, 120, 200, 300])
        del launched[:]
        ahead, _ = eng.generate(prompts, opts)
        assert any(launched) and not all(launched)              # steps fed from the device, and the prompts' steps
        monkeypatch.setattr(DeviceSampler, "can_run_ahead", staticmethod(lambda params: False))
        del launched[:]
        plain, _ = eng.generate(prompts, opts)
        assert not launched
        monkeypatch.undo()
        monkeypatch.setattr(DeviceSampler, "launch", lambda self, *a, **k: (launched.append(k.get("feed") is not None),
                                                                           real_launch(self, *a, **k))[1])
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
        assert "length" in {r.finish_reason for r in ahead} and len({r.finish_reason for r in ahead}) >= 2
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0


def test_stop_tokens_and_model_eos(models):
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams
    folder = models[("B", "float32")]
    eng = Engine.load(folder, EngineOptions(dtype="float32", max_tokens=512, max_batch=4))
    prompts = [helpers.random_tokens(n, 384, 70 + n) for n in (5, 9, 2)]
    greedy = SamplerParams(greedy=True)
    free, _ = eng.generate(prompts, GenerationOptions(max_tokens=12, ignore_eos=True, sampler=greedy))
    stop = free[0].tokens[4]
    res, _ = eng.generate(prompts, GenerationOptions(max_tokens=12, ignore_eos=True, sampler=greedy, stop_tokens=[stop]))
    for f, r in zip(free, res):
        cut = f.tokens.index(stop) if stop in f.tokens else len(f.tokens)
        assert r.tokens == f.tokens[:cut] and stop not in r.tokens
        assert r.finish_reason == ("stop" if cut < len(f.tokens) else "length")
    # the model's own eos ids (7 and 9 in this configuration) stop a request unless told otherwise
    eos = set(helpers.TINY_B["eos_token_id"])
    withstop, _ = eng.generate(prompts, GenerationOptions(max_tokens=40, sampler=greedy))
    nostop, _ = eng.generate(prompts, GenerationOptions(max_tokens=40, ignore_eos=True, sampler=greedy))
    for a, b in zip(withstop, nostop):
        hits = [i for i, t in enumerate(b.tokens) if t in eos]
        assert a.tokens == (b.tokens[:hits[0]] if hits else b.tokens)
    echo, _ = eng.generate(prompts[:1], GenerationOptions(max_tokens=3, ignore_eos=True, sampler=greedy, echo_prompt=True))
    assert echo[0].tokens[:len(prompts[0])] == prompts[0] and len(echo[0].tokens) == len(prompts[0]) + 3


@pytest.mark.parametrize("params", [dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.05, repetition_penalty=1.1),
                                    dict(temperature=1.2, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0),
                                    dict(temperature=0.6, top_k=5, top_p=1.0, min_p=0.0, repetition_penalty=1.3,
                                         presence_penalty=0.2)])
def test_sampled_generation_follows_the_chain_and_the_seed(models, params):
    """Each sampled token is what the plain chain draws from the engine's own logits with the same uniform number;
    a request draws the same alone as in a batch; another seed draws differently."""
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams
    from ziglm_b200.sampling import request_seed, uniform01
    folder = models[("A", "float32")]
    eng = Engine.load(folder, EngineOptions(dtype="float32", max_tokens=512, max_batch=4))
    prompts = [helpers.random_tokens(n, 256, 80 + n) for n in (4, 11, 6)]
    sp = SamplerParams(seed=5, **params)
    res, _ = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True, sampler=sp))
    again, _ = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True, sampler=sp))
    assert [r.tokens for r in res] == [r.tokens for r in again]
    alone, _ = eng.generate([prompts[1]], GenerationOptions(max_tokens=8, ignore_eos=True, sampler=sp))
    # request 1 of the batch has another seed than request 0 of a call of its own; the same request index draws the same
    solo_batch, _ = eng.generate([prompts[0], prompts[1]], GenerationOptions(max_tokens=8, ignore_eos=True, sampler=sp))
    assert solo_batch[1].tokens == res[1].tokens and solo_batch[0].tokens == res[0].tokens
    other, _ = eng.generate(prompts, GenerationOptions(max_tokens=8, ignore_eos=True, sampler=SamplerParams(seed=6, **params)))
    assert [r.tokens for r in other] != [r.tokens for r in res]
    cfg, w = helpers.read_folder(folder)
    mismatches = 0
    for r, (p, out) in enumerate(zip(prompts, res)):
        seq = list(p)
        for k, tok in enumerate(out.tokens):
            logits = P.forward(cfg, w, seq)[-1]
            logits = P.apply_penalties(logits, seq, sp.repetition_penalty, sp.presence_penalty, sp.repetition_penalty_window)
            want = P.sample(logits, uniform01(request_seed(5, r), k), sp.temperature, sp.top_k, sp.top_p, sp.min_p)
            mismatches += want != tok
            seq.append(tok)
    assert mismatches <= 1          # a draw that falls on a float boundary may go either way
    assert len(alone.tokens if hasattr(alone, "tokens") else alone[0].tokens) == 8


def test_command_line(models, tmp_path):
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams
    folder = models[("B", "bfloat16")]
    prompt = helpers.random_tokens(6, 384, 91)
    eng = Engine.load(folder, EngineOptions(dtype="bfloat16", max_tokens=512, max_batch=2))
    want, _ = eng.generate(prompt, GenerationOptions(max_tokens=7, ignore_eos=True, sampler=SamplerParams(greedy=True)))
    env = dict(os.environ, PYTHONPATH=ROOT)
    exe = os.path.join(ROOT, "bin", "ziglm")
    r = subprocess.run([sys.executable, exe, "run", "-m", folder, "-p", ",".join(map(str, prompt)), "-n", "7", "--greedy",
                        "--ignore-eos"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == want.tokens
    assert "Prefill:" in r.stderr and "Generation:" in r.stderr and "Total time:" in r.stderr
    r = subprocess.run([sys.executable, exe, "run", "-m", folder, "-p", " ".join(map(str, prompt)), "-n", "5", "-t", "0.9",
                        "--top-k", "20", "--seed", "3", "--echo-prompt"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr
    ids = [int(t) for t in r.stdout.split()]
    assert ids[:6] == prompt and len(ids) <= 11
    r = subprocess.run([sys.executable, exe, "bench", "-m", folder, "-n", "4"], capture_output=True, text=True, env=env,
                       timeout=300)
    assert r.returncode == 0 and r.stdout.count("Iteration") == 3, r.stderr
    sample = str(tmp_path / "sample")
    r = subprocess.run([sys.executable, exe, "test-model", "--create-sample", sample], capture_output=True, text=True,
                       env=env, timeout=300)
    assert r.returncode == 0 and os.path.exists(os.path.join(sample, "model.safetensors"))
    r = subprocess.run([sys.executable, exe, "run", "-m", sample, "-p", "1 2 3", "-n", "3", "--greedy", "--device", "cpu"],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode != 0 and "no CPU path" in r.stderr
    # a model filled from a seed, a random prompt, a stop token of the user's: the run ends at it and does not print it
    base = [sys.executable, exe, "run", "-m", "synthetic:tiny", "--random-prompt", "9", "-n", "12", "--greedy",
            "--dtype", "float32", "--seed", "4"]
    r = subprocess.run(base, capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr
    ids = [int(t) for t in r.stdout.split()]
    assert len(ids) == 12
    r = subprocess.run(base + ["--stop-ids", str(ids[5])], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and [int(t) for t in r.stdout.split()] == ids[:ids.index(ids[5])], r.stderr
    r = subprocess.run([sys.executable, exe, "bench", "-m", "synthetic:llama-1b", "--layers", "1", "-n", "3", "--batch", "3",
                        "--prompt-len", "40"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and r.stdout.count("Iteration") == 3, r.stderr
    r = subprocess.run([sys.executable, exe, "run", "-m", "synthetic:nothing", "-p", "1"], capture_output=True, text=True,
                       env=env, timeout=300)
    assert r.returncode != 0 and "not a known shape" in r.stderr
