"""The plain implementation against outputs of the reference's own CUDA kernels (tests/golden/
reference_kernels.json, made by tests/golden/make_reference_kernel_golden.py on a B200 from the reference's
unmodified src/cuda_bridge.cu).  Only kernels whose meaning coincides with the Llama architecture are there;
the model as a whole rests on the reference's formulas (its host is Zig and cannot be built here)."""
import json
import os

import torch

import plain_llama as P

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.json")))
T = lambda v, *shape: torch.as_tensor(v, dtype=torch.float32).reshape(*shape)


def close(got, want, tol=2e-6):
    want = T(want, *got.shape)
    assert torch.allclose(got, want, rtol=tol, atol=tol), (got - want).abs().max()


def test_rms_norm_is_the_reference_kernel():
    for tag in ("rmsnorm_a", "rmsnorm_b"):
        g = GOLD[tag]
        close(P.rms_norm(T(g["x"], 1, g["n"]), T(g["w"], g["n"]), g["eps"])[0], g["y"])


def test_rotation_is_the_reference_kernel():
    for tag in ("rope_full", "rope_partial"):
        g = GOLD[tag]
        inv = P.rope_inverse_frequencies(g["rot"], g["base"], None)
        # the reference forms cos and sin of a float32 angle with its GPU's sinf/cosf: a few ulp of the angle
        tol = 2e-6 if g["pos"] < 64 else 3e-5
        close(P.apply_rope(T(g["q"], 1, 3, g["hd"]), [g["pos"]], inv)[0], T(g["q_out"], 3, g["hd"]), tol)
        close(P.apply_rope(T(g["k"], 1, 1, g["hd"]), [g["pos"]], inv)[0], T(g["k_out"], 1, g["hd"]), tol)


def test_attention_of_one_token_is_the_reference_kernel():
    for tag in ("attention_all", "attention_window"):
        g = GOLD[tag]
        nh, nkv, hd = g["nh"], g["nkv"], g["hd"]
        k, v = T(g["k"], -1, nkv, hd), T(g["v"], -1, nkv, hd)
        got = P.attention_row(T(g["q"], nh, hd), k, v, g["scale"], g["window"] or None)
        close(got, T(g["o"], nh, hd), 3e-6)


def test_gated_activation_is_the_reference_kernel():
    g = GOLD["swiglu"]
    close(P.silu(T(g["gate"], 24)) * T(g["up"], 24), g["out"])


def test_matrix_vector_products_are_the_reference_kernels():
    g = GOLD["gemv_f32"]
    close(P.linear(T(g["x"], 1, 40), T(g["w"], 6, 40))[0], g["y"], 1e-5)
    g = GOLD["gemv_bf16"]
    w = T(g["w_bf16_as_float"], 6, 40).to(torch.bfloat16)          # stored with 9 decimals: exact again in bf16
    close(P.linear(T(g["x"], 1, 40), w)[0], g["y"], 1e-5)
