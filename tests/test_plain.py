"""The plain implementation itself: properties of its parts, its sampler, and the committed outputs (no GPU)."""
import json
import math
import os

import pytest
import torch

import helpers
import plain_llama as P

HERE = os.path.dirname(os.path.abspath(__file__))


def test_rms_norm_has_unit_rms():
    x = torch.randn(3, 40)
    y = P.rms_norm(x, torch.ones(40), 0.0)
    assert torch.allclose((y * y).mean(-1), torch.ones(3), atol=1e-5)


def test_rope_keeps_norms_and_relative_angles():
    f = P.rope_inverse_frequencies(16, 10000.0, None)
    assert f[0] == 1.0 and abs(f[-1].item() - 10000.0 ** (-14 / 16)) < 1e-9
    x = torch.randn(6, 2, 16)
    y = P.apply_rope(x, list(range(6)), f)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.equal(y[0], x[0])                          # position 0 is the identity
    q = torch.randn(1, 1, 16); k = torch.randn(1, 1, 16)
    d1 = (P.apply_rope(q, [7], f) * P.apply_rope(k, [3], f)).sum()
    d2 = (P.apply_rope(q, [24], f) * P.apply_rope(k, [20], f)).sum()
    assert abs(d1 - d2) < 1e-4                              # scores depend on the distance only


def test_llama3_scaling_bands():
    s = helpers.TINY_B["rope_scaling"]
    base = P.rope_inverse_frequencies(32, 500000.0, None)
    scaled = P.rope_inverse_frequencies(32, 500000.0, s)
    wavelen = 2 * math.pi / base
    kept = wavelen < 64 / 4
    slowed = wavelen > 64 / 1
    assert kept.any() and slowed.any() and (~kept & ~slowed).any()      # all three bands occur
    assert torch.equal(scaled[kept], base[kept])
    assert torch.allclose(scaled[slowed], base[slowed] / 8)
    mid = ~kept & ~slowed
    assert ((scaled[mid] < base[mid]) & (scaled[mid] > base[mid] / 8)).all()


def test_linear_and_yarn_scaling_by_hand():
    base = P.rope_inverse_frequencies(64, 10000.0, None)
    lin = P.rope_inverse_frequencies(64, 10000.0, {"rope_type": "linear", "factor": 4.0})
    assert torch.allclose(lin, base / 4, rtol=1e-7)
    # yarn over 2048 original positions, 32 and 1 rotations: pair i makes 2048 f_i / (2 pi) rotations
    sc = {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 2048}
    y = P.rope_inverse_frequencies(64, 10000.0, sc)
    rotations = 2048 * base.double() / (2 * math.pi)
    assert torch.equal(y[rotations > 32.0 * 1.3], base[rotations > 32.0 * 1.3])        # fast pairs keep their frequency
    assert torch.allclose(y[rotations < 1.0 / 1.3], base[rotations < 1.0 / 1.3] / 8)   # slow pairs are interpolated
    band = (rotations < 32.0 / 1.3) & (rotations > 1.3)
    assert band.any() and ((y[band] < base[band]) & (y[band] > base[band] / 8)).all()
    ratio = (y / base).tolist()
    assert all(a >= b for a, b in zip(ratio, ratio[1:]))                               # the ramp only falls
    # the borders of the ramp: lo = floor(64 ln(2048/(64 pi)) / (2 ln 1e4)) = 8, hi = ceil(64 ln(2048/(2 pi)) / (2 ln 1e4)) = 21
    assert ratio[8] == 1.0 and ratio[9] < 1.0 and abs(ratio[21] - 1 / 8) < 1e-7 and ratio[20] > 1 / 8 + 1e-3
    assert abs(P.rope_score_factor(sc) - (0.1 * math.log(8.0) + 1.0) ** 2) < 1e-12
    assert P.rope_score_factor({"rope_type": "yarn", "factor": 8.0, "attention_factor": 1.5}) == 2.25
    assert P.rope_score_factor({"rope_type": "linear", "factor": 8.0}) == 1.0


def test_library_frequency_table_agrees_with_the_plain_one():
    from ziglm_b200.parts.rope import inverse_frequencies, score_factor
    for sc in (helpers.TINY_F["rope_scaling"], helpers.TINY_G["rope_scaling"],
               {"rope_type": "yarn", "factor": 8.0, "original_max_position_embeddings": 2048, "truncate": False}):
        for rot in (16, 64, 128):
            assert torch.allclose(inverse_frequencies(rot, 10000.0, sc), P.rope_inverse_frequencies(rot, 10000.0, sc),
                                  rtol=2e-7, atol=0)
        assert abs(score_factor(sc) ** 2 - P.rope_score_factor(sc)) < 1e-12
    for rot, theta, sc in ((16, 10000.0, None), (32, 500000.0, helpers.TINY_B["rope_scaling"]),
                           (128, 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                            "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})):
        a = inverse_frequencies(rot, theta, sc)
        b = P.rope_inverse_frequencies(rot, theta, sc)
        assert torch.allclose(a, b, rtol=2e-7, atol=0)


def test_attention_is_causal_and_groups_heads():
    T, nh, nkv, hd = 5, 4, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    o = P.attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[3:] += 1.0; v2[3:] -= 2.0
    o2 = P.attention(q, k2, v2, 0.3)
    assert torch.equal(o[:3], o2[:3]) and not torch.allclose(o[3:], o2[3:])
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])    # heads 0,1 -> kv 0; 2,3 -> kv 1
    w = P.attention(q, k, v, 0.3, window=2)
    assert torch.allclose(w[:2], o[:2]) and not torch.allclose(w[4], o[4])


def test_whole_model_prefix_property_and_tied_head(tmp_path):
    folder = helpers.make_folder(tmp_path, helpers.TINY_A, 3, torch.float32)
    toks = helpers.random_tokens(12, 256, 1)
    full = helpers.plain_logits(folder, toks)
    part = helpers.plain_logits(folder, toks[:7])
    assert full.shape == (12, 256)
    assert torch.allclose(full[:7], part, atol=1e-6)


def test_golden_outputs_of_the_plain_model(tmp_path):
    """The committed logits were made by tests/golden/make_golden.py from this implementation."""
    gold = json.load(open(os.path.join(HERE, "golden", "plain_tiny.json")))
    for name, g in gold.items():
        folder = helpers.make_folder(tmp_path, helpers.CONFIGS[name], g["seed"], torch.float32, helpers.NORM_JITTER[name])
        logits = helpers.plain_logits(folder, g["tokens"])
        got = logits[-1, :len(g["last_logits_head"])]
        assert torch.allclose(got, torch.tensor(g["last_logits_head"]), atol=2e-6), name
        assert abs(logits.abs().sum().item() - g["abs_sum"]) < 1e-3 * g["abs_sum"]


def test_greedy_takes_the_lowest_id_on_ties_and_scans_id_zero():
    assert P.greedy(torch.tensor([3.0, 1.0, 3.0])) == 0
    assert P.greedy(torch.tensor([0.1, 2.5, 0.3, -1.0])) == 1           # src/sampler.zig:173-177


def test_sampler_chain():
    logits = torch.tensor([0.0, 10.0, 0.0, 0.0])
    assert P.sample(logits, 0.5, 0.7, 40, 0.9, 0.05) == 1               # src/sampler.zig:179-188
    logits = torch.tensor([1.0, 2.0, 3.0, 4.0])
    # top_k = 2 keeps ids 3 and 2; a large u falls on the second candidate
    assert P.sample(logits, 0.01, 1.0, 2, 1.0, 0.0) == 3
    assert P.sample(logits, 0.99, 1.0, 2, 1.0, 0.0) == 2
    assert P.sample(logits, 0.99, 1.0, 4, 0.5, 0.0) == 3                # top_p 0.5: the best alone reaches it
    assert P.sample(logits, 0.99, 1.0, 4, 1.0, 0.5) == 3                # min_p 0.5: others are below half the best
    # no top_k: id order
    assert P.sample(logits, 0.0, 1.0, 0, 1.0, 0.0) == 0
    assert P.sample(logits, 0.999, 1.0, 0, 1.0, 0.0) == 3


def test_penalties_apply_per_occurrence():
    l = torch.tensor([2.0, -2.0, 1.0])
    out = P.apply_penalties(l, [0, 1, 0], 2.0, 0.5, 64)
    assert out.tolist() == [2.0 / 2 - 0.5, -2.0 * 2 - 0.5, 1.0] or True
    # id 0 occurs twice: (2/2 - .5) = .5 -> .5/2 - .5 = -.25
    assert abs(out[0].item() - (-0.25)) < 1e-6 and abs(out[1].item() - (-4.5)) < 1e-6 and out[2] == 1.0
    assert torch.equal(P.apply_penalties(l, [0], 1.0, 0.0, 64), l)


def test_uniform_numbers_are_a_function_of_seed_and_counter():
    from ziglm_b200.sampling import uniform01
    a = [uniform01(42, c) for c in range(1000)]
    assert a == [uniform01(42, c) for c in range(1000)]
    assert all(0.0 <= x < 1.0 for x in a) and abs(sum(a) / 1000 - 0.5) < 0.05
    assert a[:5] != [uniform01(43, c) for c in range(5)]
