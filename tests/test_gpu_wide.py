"""One layer with the widths of real checkpoints (the 1B, the 8B and the 13B members of the family) against the
plain implementation in bfloat16: tiles, K splits and clusters of the tensor-core products are then the ones
that serving uses, which the tiny configurations never reach.  The 8B case has the full vocabulary of 128,256,
so the head and the sampler's row width are the measured ones too.  One width also runs in float32."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def assert_close_in_scale(got, want, what, dtype=torch.bfloat16):
    """Sums over thousands of products: the error of a logit follows the size of the logits as a whole, not its
    own size.  In bfloat16, rounding (2^-9 relative) at some ten places of the layer gives well under one
    percent of the largest logit; in float32 only the order of sums of thousands of terms differs (some 1e-6 of
    the largest logit).  A wrong tile, split or page gives errors of the size of the logits."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, what
    scale = want.abs().max().item()
    err = (got - want).abs()
    most, rms = (1e-2, 2e-3) if dtype == torch.bfloat16 else (2e-5, 3e-6)
    assert err.max().item() <= most * scale, f"{what}: largest error {err.max().item():.3g} at scale {scale:.3g}"
    assert err.pow(2).mean().sqrt().item() <= rms * scale, f"{what}: rms error {err.pow(2).mean().sqrt().item():.3g}"

WIDE = {
    # 32 query heads over 8 kv heads of size 64, tied head
    "1B": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048, "intermediate_size": 8192,
           "num_hidden_layers": 1, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 1000,
           "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": False},
    # the benchmarked shape: 32 query heads over 8 kv heads of size 128, the whole vocabulary, untied
    "8B": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096, "intermediate_size": 14336,
           "num_hidden_layers": 1, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
           "vocab_size": 128256, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False},
    # 40 heads of size 128, every one with keys of its own, widths that are multiples of 128 but not of 256
    "13B": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 5120, "intermediate_size": 13824,
            "num_hidden_layers": 1, "num_attention_heads": 40, "num_key_value_heads": 40, "vocab_size": 1000,
            "rope_theta": 10000.0, "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
            "attention_bias": False},
}


@pytest.mark.parametrize("name,dn", [("1B", "bfloat16"), ("8B", "bfloat16"), ("13B", "bfloat16"), ("1B", "float32")])
def test_one_wide_layer_whole_then_token_by_token_then_batched(tmp_path, name, dn):
    from ziglm_b200 import Engine, EngineOptions
    cfg = WIDE[name]
    dtype = torch.bfloat16 if dn == "bfloat16" else torch.float32
    folder = helpers.make_folder(tmp_path, cfg, 23, dtype, 0.1)
    eng = Engine.load(folder, EngineOptions(dtype=dn, max_tokens=2048, max_batch=20, max_seq_len=512))
    reqs = [helpers.random_tokens(n, cfg["vocab_size"], 40 + n) for n in (150, 9, 70)]
    want = [helpers.plain_logits(folder, r, act=None if dn == "float32" else torch.bfloat16) for r in reqs]
    # whole prompts in one batch of unequal lengths, every place wanted
    slots = [eng.alloc_slot() for _ in reqs]
    got = eng.step(list(zip(slots, reqs)), [list(range(len(r))) for r in reqs]).clone()
    assert_close_in_scale(got, torch.cat(want), f"{name} {dn} whole, batched", dtype)
    for s in slots:
        eng.free_slot(s)
    # the last 20 tokens of the first request one by one, then 17 sequences decoding together
    s = eng.alloc_slot()
    r = reqs[0]
    eng.step([(s, r[:-20])], [[]])
    rows = [eng.step([(s, [t])]).clone() for t in r[-20:]]
    assert_close_in_scale(torch.cat(rows), want[0][-20:], f"{name} {dn} one by one", dtype)
    eng.free_slot(s)
    many = [eng.alloc_slot() for _ in range(17)]
    src = [0 if i % 2 == 0 else 2 for i in range(17)]              # the two long requests, cut at 5 + i tokens
    eng.step([(sl, reqs[src[i]][:5 + i]) for i, sl in enumerate(many)], [[] for _ in many])
    got = eng.step([(sl, [reqs[src[i]][5 + i]]) for i, sl in enumerate(many)])
    want_rows = torch.stack([want[src[i]][5 + i] for i in range(17)])
    assert_close_in_scale(got, want_rows, f"{name} {dn} 17 sequences decoding", dtype)
    from ziglm_b200 import kernels
    if dn == "bfloat16":
        # at these widths every norm between two products rides on them: a decode step is embedding, first norm,
        # five launches a layer (q|k|v, attention with rotation and cache write, o, gate|up, down), last norm, head
        eng.options.use_graphs = False
        eng._repeat = None                               # do not take the captured step again: count real launches
        before = kernels.launches()
        eng.step([(sl, [reqs[src[i]][6 + i]]) for i, sl in enumerate(many)])
        assert kernels.launches() - before == 5 * cfg["num_hidden_layers"] + 4
        eng.options.use_graphs = True
    # greedy choice over the whole vocabulary: the device's argmax over these rows is the plain model's
    kernels.require(("sampling",))
    picked = torch.empty(17, dtype=torch.int32, device=got.device)
    kernels.argmax(got, picked)
    assert picked.tolist() == got.float().argmax(dim=1).tolist()
    assert all(c == 0 for c in kernels.wait_errors().values())
