"""The command line, in the manner of the reference's (src/cli.zig).

    ziglm run   -m <model_folder> -p "<token ids>" -n <N> [--greedy | -t T --top-k K --top-p P --min-p M --seed S]
    ziglm bench -m <model_folder> [-n N] [--batch B] [--prompt-len L]
    ziglm test-model --create-sample <folder>

``-m synthetic:<shape>`` (tiny, llama-1b, llama-8b, llama-13b, or the path of a config.json) runs a model whose
weights are filled from ``--seed`` on the device, with no folder (``--layers L`` keeps the first L layers).

Option names, defaults and meanings are the reference's (src/cli.zig:67-149): ``-m/--model``,
``-p/--prompt``, ``-n/--max-tokens`` (256), ``--max-seq-len`` (4096), ``--echo-prompt``, ``-t/--temp`` (0.7),
``--greedy`` (same as ``--temp 0``), ``--top-p`` (0.9), ``--top-k`` (40), ``--min-p`` (0.05), ``--seed`` (42),
``--gpu/--cuda`` and ``--device`` (this library runs on CUDA only), ``-j/--threads`` (accepted, unused),
``--create-sample``.  Tokenising is not part of this library, so ``--prompt`` takes token ids separated by
commas or blanks instead of text, and generated ids are printed instead of text.  ``run`` samples with a
repetition penalty of 1.1 unless greedy, and prints prefill and generation speed as the reference does
(src/cli.zig:292-334); ``bench`` runs one prompt three times greedily and prints a line per iteration
(src/cli.zig:439-469); with ``--batch B`` it generates for B prompts of ``--prompt-len`` random ids together.
``--random-prompt LEN`` stands for a prompt of LEN random ids, ``--stop-ids`` adds stop tokens to the model's
(the reference's ``stop_tokens`` option, src/engine.zig:475-482).  ``chat``, ``serve`` and ``info`` belong to the reference's tokenizer, server and GGUF
reader and do not exist here.
"""
from __future__ import annotations

import argparse
import random
import sys
from typing import List, Optional


def _ids(text: str) -> List[int]:
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"--prompt takes token ids separated by commas or blanks, found {text!r}") from None


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="ziglm", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("subcommand", choices=["run", "bench", "test-model", "help"])
    p.add_argument("-m", "--model", dest="model_path", help="path to the model folder (config.json, model.safetensors)")
    p.add_argument("-p", "--prompt", default=None, help="token ids of the prompt, separated by commas or blanks")
    p.add_argument("--prompt-file", default=None, help="a file with one prompt (token ids) per line: a batch")
    p.add_argument("-n", "--max-tokens", type=int, default=256, help="maximum tokens to generate (default: 256)")
    p.add_argument("-j", "--threads", type=int, default=None, help="accepted for compatibility, unused")
    p.add_argument("--max-seq-len", type=int, default=4096, help="maximum sequence length (default: 4096)")
    p.add_argument("--echo-prompt", action="store_true", help="print the prompt's ids before the completion")
    p.add_argument("-t", "--temp", dest="temperature", type=float, default=0.7, help="sampling temperature (default: 0.7)")
    p.add_argument("--greedy", action="store_true", help="greedy decoding (equivalent to --temp 0)")
    p.add_argument("--top-p", type=float, default=0.9, help="nucleus sampling top-p (default: 0.9)")
    p.add_argument("--top-k", type=int, default=40, help="top-k sampling (default: 40)")
    p.add_argument("--min-p", type=float, default=0.05, help="min-p sampling (default: 0.05)")
    p.add_argument("--seed", type=int, default=42, help="random seed (default: 42)")
    p.add_argument("--gpu", "--cuda", dest="use_gpu", action="store_true", help="accepted: this library always runs on CUDA")
    p.add_argument("--device", default="auto", help="cuda or auto (cpu is refused: there is no CPU path)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="precision of the run")
    p.add_argument("--max-batch", type=int, default=8, help="most sequences generated together")
    p.add_argument("--ignore-eos", action="store_true", help="do not stop at the model's end-of-sequence ids")
    p.add_argument("--random-prompt", type=int, default=None, metavar="LEN",
                   help="a prompt of LEN token ids drawn from --seed instead of -p")
    p.add_argument("--stop-ids", default=None, help="token ids that end a sequence, beside the model's own")
    p.add_argument("--layers", type=int, default=None, help="synthetic models: keep the first L layers")
    p.add_argument("--batch", type=int, default=1, help="bench: prompts generated together (default: 1)")
    p.add_argument("--prompt-len", type=int, default=20, help="bench: random ids per prompt (default: 20)")
    p.add_argument("--create-sample", dest="sample_out", default="sample_model",
                   help="test-model: folder the sample model is written to")
    return p


def _engine(args):
    from .engine import Engine, EngineOptions
    if args.device.lower() == "cpu":
        raise SystemExit("--device cpu: this library has no CPU path")
    if not args.model_path:
        raise SystemExit("a model is needed (-m <folder> or -m synthetic:<shape>)")
    print(f"Loading model: {args.model_path} ...", file=sys.stderr)
    from .config import SHAPES, read_config_json, shape
    synthetic = args.model_path.startswith("synthetic:")
    if synthetic:
        name = args.model_path[len("synthetic:"):]
        if name in SHAPES:
            cfg = shape(name)
        elif name.endswith(".json"):
            import json
            with open(name) as f:
                cfg = json.load(f)
        else:
            raise SystemExit(f"synthetic:{name}: not a known shape ({', '.join(sorted(SHAPES))}) nor a config.json")
        if args.layers:
            cfg["num_hidden_layers"] = min(args.layers, cfg["num_hidden_layers"])
    else:
        cfg = read_config_json(args.model_path)
    limit = int(cfg.get("max_position_embeddings") or args.max_seq_len)
    opts = EngineOptions(num_threads=args.threads, max_seq_len=min(args.max_seq_len, limit), seed=args.seed,
                         use_gpu=True, dtype=args.dtype, max_batch=max(args.max_batch, getattr(args, "batch", 1)))
    return Engine.from_config(cfg, opts) if synthetic else Engine.load(args.model_path, opts)


def _random_prompt(engine, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(engine.vocab_size) for _ in range(n)]


def _print_stats(stats) -> None:
    err = sys.stderr
    print("\n" + "-" * 40, file=err)
    print(f"Prefill:    {stats.prefill_tokens_per_sec():.1f} tok/s ({stats.prompt_tokens} tokens in "
          f"{stats.prefill_time_ms:.1f} ms)", file=err)
    print(f"Generation: {stats.generation_tokens_per_sec():.1f} tok/s ({stats.completion_tokens} tokens in "
          f"{stats.generation_time_ms:.1f} ms)", file=err)
    print(f"Total time: {stats.total_time_ms:.1f} ms", file=err)


def run(args) -> int:
    from .engine import GenerationOptions
    from .sampling import SamplerParams
    engine = _engine(args)
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts = [_ids(line) for line in f if line.strip()]
    elif args.prompt is not None:
        prompts = [_ids(args.prompt)]
    elif args.random_prompt:
        prompts = [_random_prompt(engine, args.random_prompt, args.seed)]
    else:
        raise SystemExit("a prompt is needed (-p \"<token ids>\", --prompt-file <file> or --random-prompt LEN)")
    greedy = args.greedy or args.temperature <= 0.0
    sampler = SamplerParams(temperature=0.0 if greedy else args.temperature, top_p=args.top_p, top_k=args.top_k,
                            min_p=args.min_p, seed=args.seed, greedy=greedy,
                            repetition_penalty=1.0 if greedy else 1.1)       # src/cli.zig:302-315
    options = GenerationOptions(max_tokens=args.max_tokens, sampler=sampler, echo_prompt=args.echo_prompt,
                                ignore_eos=args.ignore_eos, stop_tokens=_ids(args.stop_ids) if args.stop_ids else ())
    print(f"\nPrompt: {' '.join(str(t) for t in prompts[0])}" + (f" (+{len(prompts) - 1} more)" if len(prompts) > 1 else "")
          + "\n", file=sys.stderr)
    results, stats = engine.generate(prompts, options)
    for r in results:
        print(" ".join(str(t) for t in r.tokens), flush=True)
    _print_stats(stats)
    return 0


def bench(args) -> int:
    from .engine import GenerationOptions
    from .sampling import SamplerParams
    engine = _engine(args)
    print(f"Running benchmark on: {args.model_path} ...", file=sys.stderr)
    if args.prompt is not None:
        prompts = [_ids(args.prompt)] * args.batch
    else:
        # the reference's prompt has about 20 words; every sequence of a batch gets ids of its own
        n = args.random_prompt or args.prompt_len
        prompts = [_random_prompt(engine, n, args.seed + b) for b in range(args.batch)]
    options = GenerationOptions(max_tokens=args.max_tokens, ignore_eos=True,
                                sampler=SamplerParams(greedy=True, temperature=0.0, repetition_penalty=1.0))
    print("Running 3 warmup & benchmark iterations ...", file=sys.stderr)
    for it in range(3):
        _, stats = engine.generate(prompts, options)
        print(f"  Iteration {it + 1}: Prefill = {stats.prefill_tokens_per_sec():.1f} tok/s | Generation = "
              f"{stats.generation_tokens_per_sec():.1f} tok/s | Total = {stats.total_time_ms:.1f} ms")
    return 0


def test_model(args) -> int:
    """Write a small random model folder (the reference writes a 2-layer sample, src/synthetic.zig:9-18)."""
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict({
        "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 32, "max_position_embeddings": 128,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False})
    write_random_model(args.sample_out, cfg, args.seed, dtype=torch.float32)
    print(f"Sample model written to {args.sample_out}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    parser = build_parser()
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        parser.print_help()
        return 0
    args = parser.parse_args(argv)
    if args.subcommand == "run":
        return run(args)
    if args.subcommand == "bench":
        return bench(args)
    if args.subcommand == "test-model":
        return test_model(args)
    parser.print_help()
    return 0


if __name__ == "__main__":
    sys.exit(main())
