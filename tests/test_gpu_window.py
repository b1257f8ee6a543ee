"""A model with a sliding window stepped through the engine, against the plain implementation.

The window's bookkeeping gives pages back as a sequence moves on (``GroupPages.release_behind_window``), the
block table then holds -1 there, and another sequence takes the pages.  Here that happens under the real
kernels, in float32 and in bfloat16 at a head size the tensor-core attention kernels take: a prompt of more
than three pages, then decoding across more than three page boundaries, while a second sequence starts later
in pages the first one released.  Every step's logits are compared with the plain model, whose attention sees
``[p - window + 1, p]`` (the reference's range rule, src/model.zig:660-661).  In float32 the query and key
projections are doubled so that the scores are spread over several units and single keys matter: one key that
is wrongly seen or wrongly missing moves the logits.  (The head is scaled down instead, so that the logits keep
the size of about one that the comparison's tolerances are set for.)  In bfloat16 scores that large turn the
rounding of one activation into percents of a probability, in the plain model as much as in the engine, so the
projections keep their size there: a page that is released too early or a table entry of -1 that is followed
still removes or corrupts 64 keys at once, and the single key at the window's edge is planted in the kernels'
own tests (tests/test_gpu_kernels_tc.py).
"""
import dataclasses

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 128, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64, "vocab_size": 300,
    "rope_theta": 10000.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": False,
}
STD = 0.1
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def build(dn, windows, max_tokens):
    """An engine whose layer i has the window ``windows[i]`` (None: every earlier key), and its tensors."""
    from ziglm_b200 import config_from_dict
    from ziglm_b200.engine.engine import Engine, EngineOptions
    from ziglm_b200.engine.model import Model, declare_parameters
    from ziglm_b200.weights import random_tensors
    spec = config_from_dict(CFG).model_spec()
    layers = tuple(dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, window=w))
                   for layer, w in zip(spec.layers, windows))
    spec = dataclasses.replace(spec, layers=layers)
    dev = torch.device("cuda:0")
    dtype = DTYPES[dn]
    tensors = dict(random_tensors(declare_parameters(spec), 77, dtype, dev, std=STD, norm_jitter=0.1))
    for name, t in tensors.items():
        if name.endswith(("q_proj.weight", "k_proj.weight")) and dn == "float32":
            t.mul_(2.0)
        if name == "lm_head.weight":
            t.mul_(0.25)
    model = Model(spec, dtype, dev)
    model.bind(tensors)
    eng = Engine(None, model, EngineOptions(dtype=dn, max_tokens=max_tokens, max_batch=2, max_seq_len=448))
    return eng, {k: v.cpu() for k, v in tensors.items()}


def plain_logits(w, tokens, windows, act):
    """The plain model with a window per layer (the plain layer takes its window from its configuration)."""
    inv = P.rope_inverse_frequencies(CFG["head_dim"], CFG["rope_theta"], None)
    x = P.embedding(tokens, w["model.embed_tokens.weight"])
    for i, win in enumerate(windows):
        x = P.decoder_layer(dict(CFG, sliding_window=win), w, i, x, list(range(len(tokens))), inv, act)
    h = P._round(P.rms_norm(x, w["model.norm.weight"], CFG["rms_norm_eps"]), act)
    return P.linear(h, w["lm_head.weight"])


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
@pytest.mark.parametrize("windows", [(100, None), (70, 70)])
def test_windowed_layers_through_the_engine_with_pages_released_and_taken_again(dn, windows):
    eng, w = build(dn, windows, max_tokens=640)
    act = None if dn == "float32" else torch.bfloat16
    page = eng.cache.page_size
    windowed = [g for g in eng.cache.groups if g.pages.window is not None]
    assert len(eng.cache.groups) == len(set(windows)) and windowed
    a_toks = helpers.random_tokens(400, CFG["vocab_size"], 1)
    b_toks = helpers.random_tokens(170, CFG["vocab_size"], 2)
    want_a, want_b = plain_logits(w, a_toks, windows, act), plain_logits(w, b_toks, windows, act)

    a = eng.alloc_slot()
    got_a = [eng.step([(a, a_toks[:200])], [list(range(200))]).clone()]       # a prompt of more than three pages
    held_by_a = {id(g): set(p for p in g.pages.pages_of[a] if p >= 0) for g in windowed}
    got_b, b, at_b = [], None, 0
    for i in range(200, 400):                                                   # across the boundaries at 256, 320, 384
        if i == 300:
            # the second sequence starts now, in pages the first one has given back
            b = eng.alloc_slot()
            got_b.append(eng.step([(b, b_toks[:70])], [list(range(70))]).clone())
            at_b = 70
            for g in windowed:
                assert set(g.pages.pages_of[b]) & held_by_a[id(g)], "no released page was taken again"
        if b is not None and at_b < len(b_toks):
            logits = eng.step([(a, [a_toks[i]]), (b, [b_toks[at_b]])]).clone()
            got_a.append(logits[0:1]); got_b.append(logits[1:2])
            at_b += 1
        else:
            got_a.append(eng.step([(a, [a_toks[i]])]).clone())
        if i in (255, 256, 330, 399):
            eng.cache.slots.check()
            for g in windowed:
                first_visible = (i + 1) - g.pages.window + 1                    # of the next token
                row = g.pages.table[a]
                assert (row[:first_visible // page] == -1).all() and (row[first_visible // page:(i + 1 + page - 1) // page] >= 0).all()
                assert len([p for p in g.pages.pages_of[a] if p >= 0]) <= -(-g.pages.window // page) + 1
    assert at_b == len(b_toks)
    helpers.assert_close(torch.cat(got_a), want_a, DTYPES[dn], f"{dn} windows {windows}: first sequence")
    helpers.assert_close(torch.cat(got_b), want_b, DTYPES[dn], f"{dn} windows {windows}: second sequence")
    # the window is seen: the same tokens without it give other logits once positions pass it
    if windows[1] is None:
        full = plain_logits(w, a_toks[:150], (None, None), act)
        assert (full[149] - want_a[149]).abs().max() > 20 * helpers.TOL[DTYPES[dn]]["atol"]
    eng.free_slot(a); eng.free_slot(b)
    eng.cache.slots.check()
    assert all(g.pages.pool.n_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_a_windowed_prompt_in_pieces_after_pages_were_released(dn):
    """A prompt continued in pieces of several tokens once the window has already let pages go: the prompt
    kernels start at the window's first page, never at a page that is gone."""
    windows = (100, None)
    eng, w = build(dn, windows, max_tokens=448)
    act = None if dn == "float32" else torch.bfloat16
    toks = helpers.random_tokens(330, CFG["vocab_size"], 3)
    want = plain_logits(w, toks, windows, act)
    s = eng.alloc_slot()
    rows, at = [], 0
    for n in (150, 90, 3, 60, 1, 26):
        rows.append(eng.step([(s, toks[at:at + n])], [list(range(n))]).clone())
        at += n
    assert at == len(toks)
    helpers.assert_close(torch.cat(rows), want, DTYPES[dn], f"{dn} windowed prompt in pieces")
    eng.cache.slots.check()
