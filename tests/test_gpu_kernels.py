"""Each CUDA kernel alone against a plain statement of the same operation, at sizes the engine's
tiny models do not use (widths that are no power of two, odd head sizes, shuffled cache pages)."""
import math
import random

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def rnd(shape, dtype, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.fixture(scope="module")
def K():
    from ziglm_b200 import kernels
    return kernels


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(K, dtype):
    table = rnd((77, 200), dtype, seed=1)
    toks = torch.tensor([5, 76, 0, 5, 33], dtype=torch.int32)
    out = torch.empty(5, 200, dtype=torch.float32, device=DEV)
    K.embed(table.to(DEV), toks.to(DEV), out, 1.0)
    assert torch.equal(out.cpu(), P.embedding(toks.tolist(), table))
    K.embed(table.to(DEV), toks.to(DEV), out, 3.0)
    assert torch.allclose(out.cpu(), P.embedding(toks.tolist(), table) * 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_fill_gives_the_bits_of_the_host_routine(K, dtype):
    """Element i of a random tensor is the same on the device as in NumPy, for every i."""
    import numpy as np
    from ziglm_b200.weights.random_init import normal_values, random_tensor, tensor_key
    from ziglm_b200.parts.base import ParamDecl
    n = 3 * 1000 * 1000 + 17                        # more than the kernel's grid covers in one pass, an odd tail
    key = tensor_key(5, "some.tensor")
    out = torch.empty(n, dtype=dtype, device=DEV)
    K.fill_normal(out, key, 0.25, 0.5)
    z = np.concatenate([normal_values(key, s, min(1 << 16, n - s)) for s in range(0, n, 1 << 16)])
    want = torch.from_numpy(np.float32(0.25) + np.float32(0.5) * z).to(dtype)
    assert torch.equal(out.cpu(), want)
    for decl, kw in ((ParamDecl((33, 129)), dict(std=0.3)), (ParamDecl((130,), init="ones"), dict(norm_jitter=0.1)),
                     (ParamDecl((7,), init="ones"), {}), (ParamDecl((4, 4), kind="int"), {})):
        a = random_tensor("model.x", decl, 9, dtype, torch.device(DEV), **kw)
        b = random_tensor("model.x", decl, 9, dtype, torch.device("cpu"), **kw)
        assert a.dtype == b.dtype and torch.equal(a.cpu(), b)


@pytest.mark.parametrize("wd", DTYPES)
@pytest.mark.parametrize("od", DTYPES)
@pytest.mark.parametrize("d,eps", [(1000, 1e-5), (24, 1e-6), (4100, 1e-2)])
def test_rmsnorm(K, wd, od, d, eps):
    x = rnd((9, d), torch.float32, 3.0, seed=2)
    w = (1 + rnd((d,), torch.float32, 0.1, seed=3)).to(wd)
    out = torch.empty(9, d, dtype=od, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), out, eps)
    want = P.rms_norm(x, w, eps)
    assert torch.allclose(out.float().cpu(), want, **tol(od))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    out3 = torch.empty(3, d, dtype=od, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), out3, eps, rows=rows.to(DEV))
    assert torch.equal(out3.cpu(), out.cpu()[rows.long()])
    outu = torch.empty(9, d, dtype=od, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), outu, eps, weight_offset=1.0)
    assert torch.allclose(outu.float().cpu(), P.rms_norm(x, w.float() + 1.0, eps), **tol(od))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_act(K, dtype):
    T, I = 7, 203
    gu = rnd((T, 2 * I), dtype, 2.0, seed=4)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    K.gated_act(gu.to(DEV), out, "silu")
    g, u = gu[:, :I].float(), gu[:, I:].float()
    assert torch.allclose(out.float().cpu(), P.silu(g) * u, **tol(dtype))
    K.gated_act(gu.to(DEV), out, "gelu_tanh")
    want = torch.nn.functional.gelu(g, approximate="tanh") * u
    assert torch.allclose(out.float().cpu(), want, **tol(dtype))
    with pytest.raises(K.KernelError):
        K.gated_act(gu.to(DEV), out, "relu")


# ------------------------------------------------------------------------- gemm
@pytest.mark.parametrize("xd,wd,yd", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.float32, torch.bfloat16),
                                      (torch.float32, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K_", [(37, 53, 71), (1, 130, 64), (130, 1, 9), (64, 64, 16)])
def test_gemm_generic(K, xd, wd, yd, M, N, K_):
    x, w, b = rnd((M, K_), xd, seed=5), rnd((N, K_), wd, seed=6), rnd((N,), wd, seed=7)
    want = P.linear(x.float(), w, b)
    out = torch.empty(M, N, dtype=yd, device=DEV)
    K.gemm_generic(x.to(DEV), w.to(DEV), out, bias=b.to(DEV))
    assert torch.allclose(out.float().cpu(), want, **tol(yd))
    if yd == torch.float32:
        base = rnd((M, N), torch.float32, seed=8)
        acc = base.to(DEV).clone()
        K.gemm_generic(x.to(DEV), w.to(DEV), acc, accumulate=True)
        assert torch.allclose(acc.cpu(), base + P.linear(x.float(), w), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("M", [1, 2, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K_", [(130, 64), (33, 1000), (4100, 520), (31, 4), (256, 4096), (16500, 200), (20001, 36)])
def test_few_tokens_in_float32_take_the_streaming_kernel_and_keep_the_order_of_the_sums(K, M, N, K_):
    """Float operands with at most 32 tokens run a kernel of their own (32 weight rows a block, a thread per
    row and token; 128 rows a block, every warp with rows of its own, from 16,384 rows on with at most 8
    tokens).  It adds every output's products in ascending k like the tiled kernel, so the rows of a
    step of few tokens equal, bit for bit, the same rows computed inside a step of many tokens."""
    x, w, b = rnd((M, K_), torch.float32, seed=5), rnd((N, K_), torch.float32, seed=6), rnd((N,), torch.float32, seed=7)
    out = torch.full((M, N), 9.0, device=DEV)
    K.gemm_generic(x.to(DEV), w.to(DEV), out, bias=b.to(DEV))
    assert torch.allclose(out.cpu(), P.linear(x, w, b), atol=1e-5 * max(1.0, K_ ** 0.5), rtol=1e-5)
    # the same rows as the first M of 70 tokens (the tiled kernel)
    many = torch.cat([x, rnd((70 - M, K_), torch.float32, seed=8)])
    out_many = torch.empty(70, N, device=DEV)
    K.gemm_generic(many.to(DEV), w.to(DEV), out_many, bias=b.to(DEV))
    assert torch.equal(out, out_many[:M])
    # accumulating into rows of a wider buffer, inputs that are rows of a wider buffer
    wide_x = torch.zeros(M, K_ + 8, device=DEV)
    wide_x[:, 4:4 + K_] = x.to(DEV)
    wide_y = torch.full((M, N + 5), 2.0, device=DEV)
    K.gemm_generic(wide_x[:, 4:4 + K_], w.to(DEV), wide_y[:, :N], accumulate=True)
    ref = torch.full((70, N), 2.0, device=DEV)
    K.gemm_generic(many.to(DEV), w.to(DEV), ref, accumulate=True)
    assert torch.equal(wide_y[:, :N], ref[:M]) and (wide_y[:, N:] == 2.0).all()


@pytest.mark.parametrize("M,N,K_", [(97, 130, 64), (200, 257, 1000), (128, 128, 16), (300, 31, 4), (129, 640, 520)])
def test_many_tokens_in_float32_take_the_large_tiles_and_keep_the_order_of_the_sums(K, M, N, K_):
    """Float operands with more than 96 tokens run tiles of 128 x 128.  Every output is still one thread's sum in
    ascending k: rows computed there equal, bit for bit, the same rows computed 70 at a time (the 64 x 64 tiles)
    and 8 at a time (the streaming kernel); so do rows that accumulate and rows of wider buffers; unaligned rows
    fall back to the small tiles and give the same bits."""
    x, w, b = rnd((M, K_), torch.float32, seed=15), rnd((N, K_), torch.float32, seed=16), rnd((N,), torch.float32, seed=17)
    out = torch.full((M, N), 9.0, device=DEV)
    K.gemm_generic(x.to(DEV), w.to(DEV), out, bias=b.to(DEV))
    assert torch.allclose(out.cpu(), P.linear(x, w, b), atol=1e-5 * max(1.0, K_ ** 0.5), rtol=1e-5)
    for at, n in ((0, 70), (M - 70, 70), (5, 8), (M - 1, 1)):
        part = torch.empty(n, N, device=DEV)
        K.gemm_generic(x[at:at + n].to(DEV), w.to(DEV), part, bias=b.to(DEV))
        assert torch.equal(part, out[at:at + n]), (at, n)
    base = rnd((M, N + 3), torch.float32, seed=18).to(DEV)
    acc = base.clone()
    wide_x = torch.zeros(M, K_ + 8, device=DEV)
    wide_x[:, 4:4 + K_] = x.to(DEV)
    K.gemm_generic(wide_x[:, 4:4 + K_], w.to(DEV), acc[:, :N], accumulate=True)
    plain = torch.empty(M, N, device=DEV)
    K.gemm_generic(x.to(DEV), w.to(DEV), plain)
    assert torch.equal(acc[:, :N], base[:, :N] + plain) and torch.equal(acc[:, N:], base[:, N:])
    # rows that start on no 16-byte boundary: the small tiles, the same bits
    odd_x = torch.zeros(M, K_ + 8, device=DEV)
    odd_x[:, 1:1 + K_] = x.to(DEV)
    other = torch.empty(M, N, device=DEV)
    K.gemm_generic(odd_x[:, 1:1 + K_], w.to(DEV), other)
    assert torch.equal(other, plain)


def test_gemm_generic_strided_rows_and_true_float32(K):
    """Rows of a wider buffer; and float32 products are not rounded to a shorter mantissa."""
    buf = rnd((10, 100), torch.float32, seed=9).to(DEV)
    x = buf[:, 10:50]
    w = rnd((20, 40), torch.float32, seed=10)
    out = torch.empty(10, 20, device=DEV)
    K.gemm_generic(x, w.to(DEV), out)
    assert torch.allclose(out.cpu(), x.cpu() @ w.t(), atol=1e-5)
    a = torch.full((1, 8), 1.0 + 2.0 ** -20)           # needs more than a 10-bit mantissa
    bmat = torch.full((1, 8), 1.0 + 2.0 ** -21)
    o = torch.empty(1, 1, device=DEV)
    K.gemm_generic(a.to(DEV), bmat.to(DEV), o)
    exact = 8 * (1.0 + 2.0 ** -20) * (1.0 + 2.0 ** -21)
    assert abs(o.item() - exact) < 1e-6


# -------------------------------------------------------------- paged cache helpers
def paged(dense_k, dense_v, page_size, dtype, seed=0, extra_pages=3):
    """dense_[kv]: list over sequences of [len, n_kv, hd].  Returns pages in shuffled order and the table."""
    n_kv, hd = dense_k[0].shape[1:]
    need = [-(-k.shape[0] // page_size) for k in dense_k]
    total = sum(need) + extra_pages
    order = list(range(total))
    random.Random(seed).shuffle(order)
    kp = torch.full((total, n_kv, page_size, hd), 777.0, dtype=dtype)      # unwritten rows hold a poison value
    vp = torch.full((total, n_kv, page_size, hd), -777.0, dtype=dtype)
    width = max(need)
    table = torch.full((len(dense_k), width), -1, dtype=torch.int32)
    it = iter(order)
    for b, (k, v) in enumerate(zip(dense_k, dense_v)):
        for j in range(need[b]):
            p = next(it)
            table[b, j] = p
            rows = k[j * page_size:(j + 1) * page_size]
            kp[p, :, :rows.shape[0]] = rows.transpose(0, 1).to(dtype)
            vp[p, :, :rows.shape[0]] = v[j * page_size:(j + 1) * page_size].transpose(0, 1).to(dtype)
    return kp, vp, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot", [(48, 48), (48, 32), (16, 16), (128, 128)])
def test_rope_store(K, dtype, hd, rot):
    nh, nkv, page = 3, 2, 64
    lens_past, lens_new = [0, 70, 5], [9, 1, 66]
    inv = P.rope_inverse_frequencies(rot, 500000.0, None)
    T = sum(lens_new)
    qkv = rnd((T, (nh + 2 * nkv) * hd), dtype, seed=11)
    positions, seq = [], []
    for b, (p, n) in enumerate(zip(lens_past, lens_new)):
        positions += list(range(p, p + n)); seq += [b] * n
    dense = [torch.zeros(p + n, nkv, hd) for p, n in zip(lens_past, lens_new)]
    kp, vp, table = paged(dense, dense, page, dtype, seed=1)
    dq, dk, dv = qkv.to(DEV), kp.to(DEV), vp.to(DEV)
    K.rope_store(dq, nh, nkv, hd, rot, inv.to(DEV), torch.tensor(positions, dtype=torch.int32, device=DEV),
                 torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), dk, dv, page)
    q = qkv[:, :nh * hd].float().reshape(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].float().reshape(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].float().reshape(T, nkv, hd)
    qr, kr = P.apply_rope(q, positions, inv), P.apply_rope(k, positions, inv)
    got = dq.float().cpu()
    assert torch.allclose(got[:, :nh * hd].reshape(T, nh, hd), qr, **tol(dtype))
    assert torch.allclose(got[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd), kr, **tol(dtype))
    if rot < hd:
        assert torch.equal(got[:, :nh * hd].reshape(T, nh, hd)[..., rot:], q[..., rot:].to(dtype).float())
    assert torch.equal(got[:, (nh + nkv) * hd:], qkv[:, (nh + nkv) * hd:].float())       # v is left alone
    kc, vc = dk.float().cpu(), dv.float().cpu()
    for t, (pos, b) in enumerate(zip(positions, seq)):
        pg = table[b, pos // page].item()
        assert torch.allclose(kc[pg, :, pos % page], kr[t].to(dtype).float(), **tol(dtype))
        assert torch.equal(vc[pg, :, pos % page], v[t].to(dtype).float())
    # rows nobody wrote keep their content
    assert (kc == 777.0).sum() + (kc == 0.0).sum() > 0
    # no table: nothing rotates, the cache still gets k and v
    dq2, dk2, dv2 = qkv.to(DEV), kp.to(DEV), vp.to(DEV)
    K.rope_store(dq2, nh, nkv, hd, 0, None, torch.tensor(positions, dtype=torch.int32, device=DEV),
                 torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), dk2, dv2, page)
    assert torch.equal(dq2.cpu(), qkv)
    pg = table[2, 0].item()
    assert torch.equal(dk2.cpu()[pg, :, 5], qkv[lens_new[0] + lens_new[1], nh * hd:(nh + nkv) * hd].reshape(nkv, hd))


def dense_attention_case(dtype, nh, nkv, hd, lens_past, lens_new, seed):
    """Random keys/values for whole sequences, queries for the new tokens; the plain result for those."""
    ks = [rnd((p + n, nkv, hd), dtype, seed=seed + 10 * b) for b, (p, n) in enumerate(zip(lens_past, lens_new))]
    vs = [rnd((p + n, nkv, hd), dtype, seed=seed + 10 * b + 1) for b, (p, n) in enumerate(zip(lens_past, lens_new))]
    T = sum(lens_new)
    q = rnd((T, nh, hd), dtype, seed=seed + 5)
    positions, seq = [], []
    for b, (p, n) in enumerate(zip(lens_past, lens_new)):
        positions += list(range(p, p + n)); seq += [b] * n
    return ks, vs, q, positions, seq


def plain_attention_rows(ks, vs, q, positions, seq, scale, window):
    return torch.stack([P.attention_row(q[t].float(), ks[b][:pos + 1].float(), vs[b][:pos + 1].float(), scale, window)
                        for t, (pos, b) in enumerate(zip(positions, seq))])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(6, 2, 40), (4, 4, 16), (8, 1, 128), (2, 1, 256)])
@pytest.mark.parametrize("window", [None, 37])
def test_attention_general(K, dtype, nh, nkv, hd, window):
    lens_past, lens_new = [0, 130, 63, 0], [21, 1, 3, 1]
    ks, vs, q, positions, seq = dense_attention_case(dtype, nh, nkv, hd, lens_past, lens_new, seed=20)
    kp, vp, table = paged(ks, vs, 64, dtype, seed=2)
    T = q.shape[0]
    out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    # queries sit in a wider row, as they do inside the engine's q|k|v buffer
    wide = torch.zeros(T, nh * hd + 24, dtype=dtype)
    wide[:, :nh * hd] = q.reshape(T, nh * hd)
    K.attention_general(wide.to(DEV), out, nh, nkv, hd, scale, window,
                        torch.tensor(positions, dtype=torch.int32, device=DEV),
                        torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64)
    want = plain_attention_rows(ks, vs, q, positions, seq, scale, window)
    assert torch.allclose(out.float().cpu().reshape(T, nh, hd), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (6, 3, 48), (3, 3, 64), (16, 2, 256)])
@pytest.mark.parametrize("window", [None, 300])
def test_attention_general_over_many_keys_whole_and_in_parts(K, dtype, nh, nkv, hd, window):
    """Sequences of up to 1,100 keys (several parts of 256): the kernel that folds all parts of a token itself and
    the split run (a block per part, folded by a second kernel) agree bit for bit, and both with the plain rows."""
    lens_past, lens_new = [1099, 255, 256, 700, 3], [1, 1, 1, 1, 1]
    ks, vs, q, positions, seq = dense_attention_case(dtype, nh, nkv, hd, lens_past, lens_new, seed=33)
    kp, vp, table = paged(ks, vs, 64, dtype, seed=4)
    T = q.shape[0]
    scale = 1.0 / math.sqrt(hd)
    args = (nh, nkv, hd, scale, window, torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64)
    qd = q.reshape(T, nh * hd).to(DEV)
    whole = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    K.attention_general(qd, whole, *args)
    max_keys = min(1100, window or 1100)
    need = K.attention_general_scratch(T, nh, nkv, hd, max_keys)
    assert need > 0
    scratch = torch.full((need + 7,), float("nan"), device=DEV)
    parts = torch.empty_like(whole)
    K.attention_general(qd, parts, *args, max_keys=max_keys, scratch=scratch)
    assert torch.equal(parts, whole)
    # a bound on the keys that is larger than any sequence (a captured step knows only the cache's limit)
    need_big = K.attention_general_scratch(T, nh, nkv, hd, 4096)
    scratch = torch.full((need_big,), float("nan"), device=DEV)
    parts.zero_()
    K.attention_general(qd, parts, *args, max_keys=4096, scratch=scratch)
    assert torch.equal(parts, whole)
    want = plain_attention_rows(ks, vs, q, positions, seq, scale, window)
    assert torch.allclose(whole.float().cpu().reshape(T, nh, hd), want, **tol(dtype))
    # many tokens need no scratch, and too little scratch is not used
    assert K.attention_general_scratch(400, nh, nkv, hd, 1100) == 0 and K.attention_general_scratch(T, nh, nkv, hd, 200) == 0
    parts.zero_()
    K.attention_general(qd, parts, *args, max_keys=max_keys, scratch=torch.empty(8, device=DEV))
    assert torch.equal(parts, whole)


def test_attention_refuses_head_sizes_it_cannot_run(K):
    q = torch.zeros(1, 12, device=DEV)
    with pytest.raises(K.KernelError, match="head size"):
        K.attention_general(q, torch.zeros(1, 12, device=DEV), 1, 1, 12, 1.0, None,
                            torch.zeros(1, dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.zeros(1, 1, dtype=torch.int32, device=DEV), torch.zeros(1, 1, 64, 12, device=DEV),
                            torch.zeros(1, 1, 64, 12, device=DEV), 64)


# --------------------------------------------- inputs made so that a fault shows
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(K, dtype):
    """One key far back is made to dominate; the output must be its value.  A kernel that drops a block of keys,
    reads a wrong page or stops early returns something else."""
    nh, nkv, hd, n = 2, 1, 64, 700
    for far in (0, 3, 63, 64, 389, 640, 699):
        k = rnd((n, nkv, hd), dtype, 0.1, seed=30)
        v = rnd((n, nkv, hd), dtype, 1.0, seed=31)
        q = rnd((1, nh, hd), dtype, 0.1, seed=32)
        k[far] = (q[0, 0].float() * 400.0).to(dtype)        # its score towers over the rest for head 0
        kp, vp, table = paged([k], [v], 64, dtype, seed=far)
        out = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
        K.attention_general(q.reshape(1, -1).to(DEV), out, nh, nkv, hd, 1.0, None,
                            torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64)
        got = out.float().cpu().view(nh, hd)
        assert torch.allclose(got[0], v[far, 0].float(), atol=2e-2), f"far key {far}"
        want = plain_attention_rows([k], [v], q, [n - 1], [0], 1.0, None)
        assert torch.allclose(got, want[0], **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(K, dtype):
    """The dominating key sits just inside, then just outside the window."""
    nh, nkv, hd, n, window = 1, 1, 32, 200, 50
    pos = n - 1
    for offset, inside in ((window - 1, True), (window, False)):
        k = rnd((n, nkv, hd), dtype, 0.1, seed=40)
        v = rnd((n, nkv, hd), dtype, 1.0, seed=41)
        q = rnd((1, nh, hd), dtype, 0.1, seed=42)
        edge = pos - offset
        k[edge] = (q[0, 0].float() * 800.0).to(dtype)
        kp, vp, table = paged([k], [v], 64, dtype, seed=3)
        out = torch.empty(1, nh * hd, dtype=dtype, device=DEV)
        K.attention_general(q.reshape(1, -1).to(DEV), out, nh, nkv, hd, 1.0, window,
                            torch.tensor([pos], dtype=torch.int32, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64)
        got = out.float().cpu().view(hd)
        hit = torch.allclose(got, v[edge, 0].float(), atol=2e-2)
        assert hit == inside, f"key at distance {offset} inside={inside}"
        want = plain_attention_rows([k], [v], q, [pos], [0], 1.0, window)
        assert torch.allclose(got, want[0, 0], **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_reads_its_own_sequence(K, dtype):
    """Three sequences whose dominating keys hold different values: each must return its own."""
    nh, nkv, hd = 2, 2, 16
    lens = [90, 64, 129]
    ks, vs, qs = [], [], []
    for b, n in enumerate(lens):
        k = rnd((n, nkv, hd), dtype, 0.1, seed=50 + b)
        v = rnd((n, nkv, hd), dtype, 1.0, seed=60 + b)
        q = rnd((1, nh, hd), dtype, 0.1, seed=70 + b)
        k[n // 2, 0] = (q[0, 0].float() * 900.0).to(dtype)
        k[n // 3, 1] = (q[0, 1].float() * 900.0).to(dtype)
        ks.append(k); vs.append(v); qs.append(q)
    kp, vp, table = paged(ks, vs, 64, dtype, seed=4)
    q = torch.cat(qs)
    out = torch.empty(3, nh * hd, dtype=dtype, device=DEV)
    K.attention_general(q.reshape(3, -1).to(DEV), out, nh, nkv, hd, 1.0, None,
                        torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV),
                        torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64)
    got = out.float().cpu().view(3, nh, hd)
    for b, n in enumerate(lens):
        assert torch.allclose(got[b, 0], vs[b][n // 2, 0].float(), atol=2e-2)
        assert torch.allclose(got[b, 1], vs[b][n // 3, 1].float(), atol=2e-2)


# -------------------------------------------------------------------- sampling
def test_argmax(K):
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(5, 1000, generator=g)
    logits[1, 400] = logits[1, 17] = 9.0                   # a tie: the lower id wins
    logits[2, 0] = 50.0                                    # id 0 is a candidate like any other
    logits[3, 999] = 50.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    K.argmax(logits.to(DEV), out)
    assert out.tolist() == [P.greedy(r) for r in logits]
    assert out[1] == 17 and out[2] == 0 and out[3] == 999
    wide = torch.randn(3, 130000, generator=g)
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    K.argmax(wide.to(DEV), out)
    assert out.tolist() == wide.argmax(-1).tolist()


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [(0.7, 40, 0.9, 0.05), (1.0, 0, 1.0, 0.0), (1.3, 5, 1.0, 0.0),
                                                           (0.5, 0, 1.0, 0.1), (1.0, 1000, 0.95, 0.0),
                                                           (1.0, 0, 0.9, 0.0), (0.6, 0, 0.5, 0.02), (2.5, 0, 0.97, 0.0)])
def test_sample_follows_the_chain(K, temperature, top_k, top_p, min_p):
    from ziglm_b200.sampling import uniform01
    V, rows = 331, 48
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(rows, V, generator=g) * 3.0
    rng = torch.tensor([[1234 + r, r * 3] for r in range(rows)], dtype=torch.int64)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample(logits.to(DEV), out, rng.to(DEV), temperature, top_k, top_p, min_p)
    want = [P.sample(logits[r], uniform01(1234 + r, r * 3), temperature, top_k, top_p, min_p) for r in range(rows)]
    got = out.tolist()
    assert sum(a != b for a, b in zip(got, want)) <= 1, (got, want)     # a draw on a float boundary may differ
    # a row draws the same alone as in the batch
    solo = torch.empty(1, dtype=torch.int32, device=DEV)
    K.sample(logits[7:8].to(DEV), solo, rng[7:8].to(DEV), temperature, top_k, top_p, min_p)
    assert solo.item() == got[7]


def test_sample_with_changing_row_counts_and_a_wide_vocabulary(K):
    """The sampler keeps scratch between calls: calls with 1, 40, 3 and 40 rows, one after another, must each
    give the plain draw.  The vocabulary is wide enough that a row is cut into slices over several blocks."""
    from ziglm_b200.sampling import uniform01
    V, most = 12007, 40
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(most, V, generator=g) * 2.0
    rng = torch.tensor([[77 + 5 * r, r] for r in range(most)], dtype=torch.int64)
    hist = torch.randint(0, V, (most, 64), generator=g, dtype=torch.int32)
    want = []
    for r in range(most):
        row = P.apply_penalties(logits[r], hist[r].tolist(), 1.1, 0.0, 64)
        want.append(P.sample(row, uniform01(77 + 5 * r, r), 0.8, 40, 0.95, 0.02))
    for rows in (1, most, 3, most):
        d = logits[:rows].to(DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        K.sample(d, out, rng[:rows].to(DEV), 0.8, 40, 0.95, 0.02, 1.1, 0.0, hist[:rows].to(DEV))
        got = out.tolist()
        assert sum(a != b for a, b in zip(got, want)) <= (1 if rows > 8 else 0), (rows, got, want[:rows])


def test_sample_distribution_and_ties(K):
    V, n = 6, 4000
    logits = torch.tensor([0.0, 1.0, 2.0, 0.5, -1.0, 2.0]).repeat(n, 1)
    rng = torch.tensor([[99, c] for c in range(n)], dtype=torch.int64)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    K.sample(logits.to(DEV), out, rng.to(DEV), 1.0, 0, 1.0, 0.0)
    freq = torch.bincount(out.cpu().long(), minlength=V).float() / n
    p = torch.softmax(logits[0], -1)
    assert (freq - p).abs().max() < 0.03
    K.sample(logits.to(DEV), out, rng.to(DEV), 1.0, 2, 1.0, 0.0)           # ids 2 and 5 tie for the top
    assert set(out.tolist()) == {2, 5}
    K.sample(torch.zeros(n, V).to(DEV), out, rng.to(DEV), 1.0, 3, 1.0, 0.0)   # all equal: the three lowest ids
    assert set(out.tolist()) == {0, 1, 2}


def test_sample_penalties(K):
    logits = torch.tensor([[2.0, -2.0, 1.0, 0.0]])
    hist = torch.tensor([[-1, 0, 1, 0]], dtype=torch.int32)
    d = logits.to(DEV)
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    K.sample(d, out, torch.tensor([[1, 1]], dtype=torch.int64, device=DEV), 1.0, 0, 1.0, 0.0, 2.0, 0.5, hist.to(DEV))
    want = P.apply_penalties(logits[0], [0, 1, 0], 2.0, 0.5, 64)
    assert torch.allclose(d.cpu()[0], want)


def test_top_p_without_top_k_keeps_the_nucleus_of_the_sorted_chain(K):
    """top_p with no top_k: the kept set is the shortest prefix by descending probability that reaches top_p, also
    when that takes more candidates than any top_k this library sorts (a flat row of a wide vocabulary), with
    equal logits at the edge taken in id order; nothing outside the set is ever drawn."""
    from ziglm_b200.sampling import uniform01
    V = 50021
    g = torch.Generator().manual_seed(21)
    flat = torch.randn(V, generator=g) * 0.3                           # the nucleus of 0.9 holds tens of thousands
    peaked = torch.randn(V, generator=g) * 4.0
    ties = torch.zeros(V)
    ties[100:140] = 5.0                                                # 40 equal logits: top_p cuts among them
    rows = torch.stack([flat, peaked, ties])
    for top_p in (0.9, 0.3):
        prob = torch.softmax(rows, -1)
        for r in range(3):
            order = sorted(range(V), key=lambda i: (-prob[r, i].item(), i))
            cum, nucleus = 0.0, set()
            for i in order:
                nucleus.add(i); cum += prob[r, i].item()
                if cum >= top_p:
                    break
            picks = set()
            for c in range(24):
                rng = torch.tensor([[77 + r, c]], dtype=torch.int64, device=DEV)
                out = torch.empty(1, dtype=torch.int32, device=DEV)
                K.sample(rows[r:r + 1].to(DEV), out, rng, 1.0, 0, top_p, 0.0)
                want = P.sample(rows[r], uniform01(77 + r, c), 1.0, 0, top_p, 0.0)
                # the draw is a running sum over the kept ids: over tens of thousands of equal probabilities (the
                # third row) the device's order of additions may end one id away from the sequential sum
                assert out.item() == want if r < 2 else abs(out.item() - want) <= 2
                picks.add(out.item())
            # a float boundary may move the set's edge by one id; nothing far outside is drawn
            assert len(picks - nucleus) <= 1 and len(picks) > 1


def test_sample_refuses_what_it_cannot_do(K):
    l = torch.zeros(1, 10, device=DEV)
    o = torch.empty(1, dtype=torch.int32, device=DEV)
    r = torch.zeros(1, 2, dtype=torch.int64, device=DEV)
    with pytest.raises(K.KernelError, match="1024"):
        K.sample(l, o, r, 1.0, 5000, 1.0, 0.0)
    with pytest.raises(K.KernelError, match="temperature"):
        K.sample(l, o, r, 0.0)
    with pytest.raises(K.KernelError, match="on the device"):
        K.argmax(torch.zeros(1, 10), o)
