"""Writes tests/golden/reference_kernels.json: outputs of the reference's own CUDA kernels on small inputs.

The reference's model code is Zig and cannot be compiled here, but its CUDA file (src/cuda_bridge.cu) compiles
unchanged with nvcc.  This script runs, on a GPU, the kernels whose meaning coincides with the Llama
architecture (RMSNorm, rotation of pairs (i, i + rot/2) with theta = pos / base^(2i/rot), attention of one
token over a float32 cache with and without a window, silu(gate) * up, the bf16 and float32 matrix-vector
products) and stores inputs and outputs.  tests/test_reference_golden.py compares the plain implementation
with them on the CPU.

    nvcc -shared -Xcompiler -fPIC -gencode arch=compute_100a,code=sm_100a -O3 -o libziglm_cuda.so <reference>/src/cuda_bridge.cu
    python tests/golden/make_reference_kernel_golden.py path/to/libziglm_cuda.so
"""
import ctypes
import json
import os
import sys
from ctypes import c_float, c_int, c_void_p

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
lib = ctypes.CDLL(sys.argv[1])
P = c_void_p
for name, argtypes in {
    "cuda_gemv_bf16": [P, P, P, c_int, c_int, P],
    "cuda_gemv_f32": [P, P, P, c_int, c_int, P],
    "cuda_rmsnorm": [P, P, P, c_int, c_float, c_int, P],
    "cuda_rope": [P, P, c_int, c_int, c_int, c_int, c_int, c_float, P],
    "cuda_attention_forward": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, P],
    "cuda_swiglu": [P, P, P, c_int, P],
}.items():
    fn = getattr(lib, name)
    fn.argtypes, fn.restype = argtypes, None

dev = "cuda:0"
gen = torch.Generator().manual_seed(2024)
rnd = lambda *shape: torch.randn(*shape, generator=gen)
lst = lambda t: [round(float(v), 9) for v in t.flatten().tolist()]
p = lambda t: t.data_ptr()
out = {}

# RMSNorm: n = 40, eps = 1e-5 (and a second one with another eps)
for tag, n, eps in (("rmsnorm_a", 40, 1e-5), ("rmsnorm_b", 56, 1e-6)):
    x, w = rnd(n), 1.0 + 0.1 * rnd(n)
    y = torch.empty(n, device=dev)
    xd, wd = x.to(dev), w.to(dev)
    lib.cuda_rmsnorm(p(xd), p(wd), p(y), n, eps, 0, None)
    torch.cuda.synchronize()
    out[tag] = {"n": n, "eps": eps, "x": lst(x), "w": lst(w), "y": lst(y.cpu())}

# rotation: 3 query heads, 1 kv head, head size 16, two rotated widths
for tag, hd, rot, pos, base in (("rope_full", 16, 16, 7, 10000.0), ("rope_partial", 16, 8, 131, 500000.0)):
    q, k = rnd(3, hd), rnd(1, hd)
    qd, kd = q.clone().to(dev), k.clone().to(dev)
    lib.cuda_rope(p(qd), p(kd), pos, 3, 1, hd, rot, base, None)
    torch.cuda.synchronize()
    out[tag] = {"hd": hd, "rot": rot, "pos": pos, "base": base, "q": lst(q), "k": lst(k), "q_out": lst(qd.cpu()),
                "k_out": lst(kd.cpu())}

# attention of the token at position 9: 4 heads, 2 kv heads, head size 8; all keys, then a window of 4
for tag, window in (("attention_all", 0), ("attention_window", 4)):
    nh, nkv, hd, pos = 4, 2, 8, 9
    q, k, v = rnd(nh, hd), rnd(pos + 1, nkv, hd), rnd(pos + 1, nkv, hd)
    o = torch.empty(nh * hd, device=dev)
    qd, kd, vd = q.to(dev), k.reshape(pos + 1, nkv * hd).contiguous().to(dev), v.reshape(pos + 1, nkv * hd).contiguous().to(dev)
    scale = 1.0 / hd ** 0.5
    lib.cuda_attention_forward(p(qd), p(kd), p(vd), p(o), 0, pos, pos + 1, nh, nkv, hd, nkv * hd, scale, 0.0, window, None)
    torch.cuda.synchronize()
    out[tag] = {"nh": nh, "nkv": nkv, "hd": hd, "window": window, "scale": scale, "q": lst(q), "k": lst(k), "v": lst(v),
                "o": lst(o.cpu())}

# silu(gate) * up
g, u = 3.0 * rnd(24), rnd(24)
a = torch.empty(24, device=dev)
gd, ud = g.to(dev), u.to(dev)
lib.cuda_swiglu(p(gd), p(ud), p(a), 24, None)
torch.cuda.synchronize()
out["swiglu"] = {"gate": lst(g), "up": lst(u), "out": lst(a.cpu())}

# matrix-vector products: weights [6, 40] in float32 and in bf16
w, x = rnd(6, 40), rnd(40)
y = torch.empty(6, device=dev)
wd, xd = w.to(dev), x.to(dev)
lib.cuda_gemv_f32(p(wd), p(xd), p(y), 6, 40, None)
torch.cuda.synchronize()
out["gemv_f32"] = {"w": lst(w), "x": lst(x), "y": lst(y.cpu())}
wb = w.to(torch.bfloat16)
wbd = wb.to(dev)
lib.cuda_gemv_bf16(p(wbd), p(xd), p(y), 6, 40, None)
torch.cuda.synchronize()
out["gemv_bf16"] = {"w_bf16_as_float": lst(wb.float()), "x": lst(x), "y": lst(y.cpu())}

json.dump(out, open(os.path.join(HERE, "reference_kernels.json"), "w"), indent=0)
print("wrote", len(out), "cases")
