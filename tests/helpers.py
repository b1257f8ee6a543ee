"""Shared by the tests: the two tiny configurations, model folders, the plain model's logits."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional, Sequence

import torch

# Two configurations of the architecture that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256,
    "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": False,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": True,
    "eos_token_id": [7, 9],
}
# A third one with awkward sizes: widths and a vocabulary that are no power of two, head size 48.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 120, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "vocab_size": 331,
    "rope_theta": 10000.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": False,
}
# Two with the head sizes the tensor-core attention kernels take (64 and 128): grouped heads with an even and
# with an odd group, a feed-forward width that is no multiple of a tile, biases and llama3 scaling in one.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 256, "intermediate_size": 688, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 500,
    "rope_theta": 10000.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": False,
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 384, "intermediate_size": 512, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 128, "vocab_size": 300,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "attention_bias": True,
}
# Two with what config.json allows beyond the usual checkpoints: biases in the feed-forward with the linear
# stretching of positions (head size 64, so that bfloat16 takes the tensor-core kernels and the gated product
# adds its biases in the epilogue), and the yarn stretching with every head its own key/value head.
TINY_F = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 192, "intermediate_size": 328, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 64, "vocab_size": 411,
    "rope_theta": 10000.0, "rope_scaling": {"rope_type": "linear", "factor": 4.0},
    "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "attention_bias": False, "mlp_bias": True,
}
TINY_G = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 128, "intermediate_size": 136, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 200,
    "rope_theta": 10000.0,
    "rope_scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64,
                     "beta_fast": 8.0, "beta_slow": 1.0},
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "attention_bias": True, "mlp_bias": True,
}
# One with a sliding window in every layer (position p sees the 48 positions up to p), at a head size the
# tensor-core attention kernels take: prompts longer than the window, pages given back while decoding.
TINY_H = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 256, "intermediate_size": 344, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 320,
    "rope_theta": 10000.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": False, "sliding_window": 48,
}
NORM_JITTER = {"A": 0.0, "B": 0.1, "C": 0.1, "D": 0.1, "E": 0.1, "F": 0.1, "G": 0.1, "H": 0.1}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F, "G": TINY_G, "H": TINY_H}


def make_folder(tmp_path, cfg: dict, seed: int, dtype: torch.dtype, norm_jitter: float = 0.0, std: float = 0.02) -> str:
    from ziglm_b200 import config_from_dict, write_random_model
    tag = f"{cfg['hidden_size']}x{cfg['num_hidden_layers']}x{cfg['vocab_size']}"
    folder = os.path.join(str(tmp_path), f"model_{tag}_{seed}_{str(dtype).split('.')[-1]}_{norm_jitter}_{std}")
    # the values are the same wherever they are computed; a GPU is only faster for the wide models
    device = "cuda" if torch.cuda.is_available() else "cpu"
    write_random_model(folder, config_from_dict(cfg), seed, dtype=dtype, std=std, norm_jitter=norm_jitter,
                       device=device)
    return folder


def read_folder(folder: str):
    """config.json as a dictionary and the tensors by name, read with the safetensors package
    (not with the library's own reader)."""
    from safetensors.torch import load_file
    cfg = json.load(open(os.path.join(folder, "config.json")))
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def plain_logits(folder: str, tokens: Sequence[int], act: Optional[torch.dtype] = None) -> torch.Tensor:
    import plain_llama
    cfg, w = read_folder(folder)
    return plain_llama.forward(cfg, w, list(tokens), act=act)


# Tolerances, fixed once.  float32: the engine and the plain model differ in the order of
# float32 sums only (logits here are of size 0.1 to 1).  bfloat16: the plain model rounds
# activations at the same places; what is left is the order of sums, the rounding of
# probabilities inside the tensor-core attention and values that round the other way.
TOL = {torch.float32: dict(atol=2e-5, rtol=1e-4), torch.bfloat16: dict(atol=1.5e-2, rtol=2e-2)}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float32)
    want = want.detach().to("cpu", torch.float32)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    tol = TOL[dtype]
    err = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    bad = err > bound
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {bad.numel()} values differ; first at {idx}: got {got[tuple(idx)].item():.6g}, "
            f"want {want[tuple(idx)].item():.6g}; largest error {err.max().item():.3g} "
            f"(scale {want.abs().max().item():.3g})")
