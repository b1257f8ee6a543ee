"""One layer with the widths of real checkpoints (the 1B and the 13B members of the family) against the plain
implementation in bfloat16: tiles, K splits and clusters of the tensor-core products are then the ones that
serving uses, which the tiny configurations never reach."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def assert_close_in_scale(got, want, what):
    """Sums over thousands of bf16 products: the error of a logit follows the size of the logits as a whole,
    not its own size.  Rounding to bf16 (2^-9 relative) at some ten places of the layer gives well under one
    percent of the largest logit; a wrong tile, split or page gives errors of the size of the logits."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, what
    scale = want.abs().max().item()
    err = (got - want).abs()
    assert err.max().item() <= 1e-2 * scale, f"{what}: largest error {err.max().item():.3g} at scale {scale:.3g}"
    assert err.pow(2).mean().sqrt().item() <= 2e-3 * scale, f"{what}: rms error {err.pow(2).mean().sqrt().item():.3g}"

WIDE = {
    # 32 query heads over 8 kv heads of size 64, tied head
    "1B": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048, "intermediate_size": 8192,
           "num_hidden_layers": 1, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 1000,
           "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": False},
    # 40 heads of size 128, every one with keys of its own, widths that are multiples of 128 but not of 256
    "13B": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 5120, "intermediate_size": 13824,
            "num_hidden_layers": 1, "num_attention_heads": 40, "num_key_value_heads": 40, "vocab_size": 1000,
            "rope_theta": 10000.0, "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
            "attention_bias": False},
}


@pytest.mark.parametrize("name", ["1B", "13B"])
def test_one_wide_layer_whole_then_token_by_token_then_batched(tmp_path, name):
    from ziglm_b200 import Engine, EngineOptions
    cfg = WIDE[name]
    folder = helpers.make_folder(tmp_path, cfg, 23, torch.bfloat16, 0.1)
    eng = Engine.load(folder, EngineOptions(dtype="bfloat16", max_tokens=2048, max_batch=20, max_seq_len=512))
    reqs = [helpers.random_tokens(n, cfg["vocab_size"], 40 + n) for n in (150, 9, 70)]
    want = [helpers.plain_logits(folder, r, act=torch.bfloat16) for r in reqs]
    # whole prompts in one batch of unequal lengths, every place wanted
    slots = [eng.alloc_slot() for _ in reqs]
    got = eng.step(list(zip(slots, reqs)), [list(range(len(r))) for r in reqs]).clone()
    assert_close_in_scale(got, torch.cat(want), f"{name} whole, batched")
    for s in slots:
        eng.free_slot(s)
    # the last 20 tokens of the first request one by one, then 17 sequences decoding together
    s = eng.alloc_slot()
    r = reqs[0]
    eng.step([(s, r[:-20])], [[]])
    rows = [eng.step([(s, [t])]).clone() for t in r[-20:]]
    assert_close_in_scale(torch.cat(rows), want[0][-20:], f"{name} one by one")
    eng.free_slot(s)
    many = [eng.alloc_slot() for _ in range(17)]
    src = [0 if i % 2 == 0 else 2 for i in range(17)]              # the two long requests, cut at 5 + i tokens
    eng.step([(sl, reqs[src[i]][:5 + i]) for i, sl in enumerate(many)], [[] for _ in many])
    got = eng.step([(sl, [reqs[src[i]][5 + i]]) for i, sl in enumerate(many)])
    want_rows = torch.stack([want[src[i]][5 + i] for i in range(17)])
    assert_close_in_scale(got, want_rows, f"{name} 17 sequences decoding")
    from ziglm_b200 import kernels
    assert kernels.gemm_tc_status() == 0 and kernels.attention_tc_status() == 0 and kernels.attention_fmha_status() == 0
