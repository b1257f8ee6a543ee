"""Sizes that the configuration allows and no checkpoint of the family has: every head size in steps of 16 up
to 256, one key/value head for seven or seventeen query heads, every head its own, widths that are no multiple
of eight (rows of bfloat16 weights then start on no 16-byte boundary, which the tensor-core products' copies
need), a vocabulary of two, heads of which only a part is rotated.  Each runs prompts of unequal lengths in one step and then five tokens each, in
float32 and in bfloat16, against the plain implementation: a kernel takes the size or hands it to one that does,
never a wrong result."""
import warnings

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def cfg(hidden, inter, heads, kv, head_dim, vocab, layers=2, tie=False, bias=False, mlp_bias=False, **more):
    return {**more, "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": hidden,
            "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": kv, "head_dim": head_dim, "vocab_size": vocab, "rope_theta": 10000.0,
            "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "tie_word_embeddings": tie,
            "attention_bias": bias, "mlp_bias": mlp_bias}


ODD = {
    "width 100, 173; 5 heads of 16, each its own; 257 ids": cfg(100, 173, 5, 5, 16, 257),
    "7 heads of 80 on one key/value head": cfg(136, 300, 7, 1, 80, 1001, bias=True),
    "heads of 96, tied": cfg(200, 344, 6, 2, 96, 513, tie=True),
    "heads of 112, 99 ids": cfg(224, 100, 2, 2, 112, 99),
    "heads of 160": cfg(320, 264, 4, 1, 160, 777),
    "heads of 256, feed-forward biases": cfg(256, 520, 2, 1, 256, 300, mlp_bias=True),
    "17 heads of 64 on a key/value head": cfg(128, 256, 34, 2, 64, 300),
    "width 72, 77; 31 ids": cfg(72, 77, 3, 3, 32, 31),
    "9 heads of 64 in groups of 3; 4097 ids": cfg(264, 1000, 9, 3, 64, 4097),
    "5 heads of 128, each its own; 50001 ids": cfg(520, 1384, 5, 5, 128, 50001, layers=1),
    "width 1, two ids": cfg(1, 1, 1, 1, 16, 2),
    # part of a head rotated (pairs (i, i + rot/2) of its first rot elements, the rest as it is): 32 of 64 and 32 of
    # 128 (the decode kernel rotates them itself), 24 of 48 (the rotation kernel)
    "half of a head of 64 rotated": cfg(256, 344, 4, 2, 64, 300, partial_rotary_factor=0.5),
    "a quarter of a head of 128 rotated": cfg(384, 512, 3, 1, 128, 300, partial_rotary_factor=0.25,
                                             rope_parameters={"rope_type": "linear", "factor": 2.0, "rope_theta": 50000.0}),
    "half of a head of 48 rotated": cfg(144, 200, 3, 3, 48, 211, partial_rotary_factor=0.5),
    # the tanh form of gelu in the gate's place, with biases; at a head size and width that take the fused product
    "gelu gate": cfg(256, 344, 4, 2, 64, 300, mlp_bias=True, hidden_act="gelu_pytorch_tanh"),
    "gelu gate, narrow": cfg(72, 77, 3, 3, 32, 31, hidden_act="gelu_pytorch_tanh"),
}


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ODD))
def test_odd_sizes_prompts_then_tokens(tmp_path, name, dn):
    from ziglm_b200 import Engine, EngineOptions
    c = ODD[name]
    dtype = torch.float32 if dn == "float32" else torch.bfloat16
    folder = helpers.make_folder(tmp_path, c, 5, dtype, 0.1)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)       # bfloat16 at these head sizes: the plain attention kernel
        eng = Engine.load(folder, EngineOptions(dtype=dn, max_tokens=1024, max_batch=4, max_seq_len=400))
    reqs = [helpers.random_tokens(n, c["vocab_size"], 10 + n) for n in (150, 7, 66)]
    want = [helpers.plain_logits(folder, r, act=None if dn == "float32" else torch.bfloat16) for r in reqs]
    slots = [eng.alloc_slot() for _ in reqs]
    cut = [len(r) - 5 for r in reqs]
    got = eng.step([(s, r[:k]) for s, r, k in zip(slots, reqs, cut)], [list(range(k)) for k in cut]).clone()
    helpers.assert_close(got, torch.cat([w[:k] for w, k in zip(want, cut)]), dtype, f"{name} {dn}: prompts")
    for j in range(5):
        got = eng.step([(s, [r[k + j]]) for s, r, k in zip(slots, reqs, cut)]).clone()
        helpers.assert_close(got, torch.stack([w[k + j] for w, k in zip(want, cut)]), dtype, f"{name} {dn}: token {j}")
    for s in slots:
        eng.free_slot(s)
    eng.cache.slots.check()
    from ziglm_b200 import kernels
    assert all(v == 0 for v in kernels.wait_errors().values())
