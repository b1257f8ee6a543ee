"""config.json dictionaries of a few members of the Llama family, for models with random weights.

The reference's ``synthetic`` stage writes one fixed 2-layer sample (src/synthetic.zig:9-18); these are the
shapes the measurements of this library name, so that the command line and ``bench.py`` agree on them.
No checkpoint is read: ``Engine.from_config`` fills the weights from a seed.
"""
from __future__ import annotations

import copy
from typing import Any, Dict


def _llama3(factor: float) -> Dict[str, Any]:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 8192}


SHAPES: Dict[str, Dict[str, Any]] = {
    # the reference's sample model (src/synthetic.zig:9-18)
    "tiny": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 32,
        "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 128, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False, "attention_bias": False,
    },
    "llama-1b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
        "rope_theta": 500000.0, "rope_scaling": _llama3(32.0), "max_position_embeddings": 131072,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": False,
    },
    "llama-8b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
        "rope_theta": 500000.0, "rope_scaling": _llama3(8.0), "max_position_embeddings": 131072,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False,
    },
    "llama-13b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": 5120, "intermediate_size": 13824, "num_hidden_layers": 40,
        "num_attention_heads": 40, "num_key_value_heads": 40, "head_dim": 128, "vocab_size": 32000,
        "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 4096,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False,
    },
}


def shape(name: str) -> Dict[str, Any]:
    """A copy of the named config.json dictionary."""
    try:
        return copy.deepcopy(SHAPES[name])
    except KeyError:
        raise KeyError(f"no shape named {name!r} (known: {', '.join(sorted(SHAPES))})") from None
