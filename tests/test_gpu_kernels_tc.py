"""The tensor-core kernels alone (tcgen05/TMA matrix product, paged attention for prompts and for decode
steps) against plain float32 statements of the same operations, at sizes other than the engine's."""
import math

import pytest
import torch

import plain_llama as P
from test_gpu_kernels import DEV, dense_attention_case, paged, plain_attention_rows, rnd

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def K():
    from ziglm_b200 import kernels
    return kernels


def ref_product(x, w, b=None):
    return P.linear(x.float(), w, b)


# every token-tile width (16..256), one tile and many, K with a ragged tail, N that is no multiple of 128
@pytest.mark.parametrize("T,N,K_", [(1, 331, 120), (8, 256, 512), (16, 128, 64), (17, 1000, 264), (45, 128, 64),
                                    (64, 4096, 1024), (70, 352, 64), (128, 20000, 192), (300, 1000, 4096),
                                    (1000, 40000, 128)])
@pytest.mark.parametrize("out_dtype", [BF, torch.float32])
def test_gemm_tc_shapes(K, T, N, K_, out_dtype):
    x, w, b = rnd((T, K_), BF, seed=1), rnd((N, K_), BF, 0.05, seed=2), rnd((N,), BF, seed=3)
    want = ref_product(x, w, b)
    out = torch.full((T, N), 7.0, dtype=out_dtype, device=DEV)
    assert K.gemm_tc(x.to(DEV), w.to(DEV), out, bias=b.to(DEV))
    torch.cuda.synchronize()
    assert K.gemm_tc_status() == 0
    tol = dict(atol=1e-3, rtol=1e-3) if out_dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(out.float().cpu(), want, **tol)


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("T", [1, 8, 33, 41, 64])
def test_gemm_tc_split_k_is_exact_in_order(K, splits, T):
    """K split over the CTAs of a cluster: same result whatever the number of splits, up to the order of float sums;
    and the same bits every time."""
    x, w = rnd((T, 2048), BF, seed=4), rnd((256, 2048), BF, 0.05, seed=5)
    base = rnd((T, 256), torch.float32, seed=6)
    out = base.to(DEV).clone()
    assert K.gemm_tc(x.to(DEV), w.to(DEV), out, accumulate=True, splits=splits)
    again = base.to(DEV).clone()
    assert K.gemm_tc(x.to(DEV), w.to(DEV), again, accumulate=True, splits=splits)
    torch.cuda.synchronize()
    assert K.gemm_tc_status() == 0
    assert torch.equal(out, again)
    assert torch.allclose(out.cpu(), base + ref_product(x, w), atol=2e-3, rtol=1e-3)


# Steps of more than 128 tokens: the kernel that pairs two CTAs on tiles of 256 weight rows (splits=0) and the
# one-CTA kernel (splits=1), in every output mode.  Shapes: one pair tile; an odd number of row tiles (the last
# pair is half empty); a ragged K and N; many tiles per pair and a long K; few tiles and a long K (the
# accumulating product is then also cut along K: 4 and 8 parts, the last part shorter).
@pytest.mark.parametrize("splits", [0, 1])
@pytest.mark.parametrize("T,N,K_", [(129, 256, 64), (300, 1000, 4096), (1000, 40000, 128), (600, 392, 200),
                                    (2050, 6144, 1024), (256, 4096, 14336), (200, 2048, 1000)])
def test_gemm_tc_prompt_tiles_on_one_cta_and_on_a_pair(K, splits, T, N, K_):
    x, w, b = rnd((T, K_), BF, seed=21), rnd((N, K_), BF, 0.05, seed=22), rnd((N,), BF, seed=23)
    want = ref_product(x, w, b)
    dx, dw, db = x.to(DEV), w.to(DEV), b.to(DEV)
    for out_dtype in (BF, torch.float32):
        out = torch.full((T, N), 7.0, dtype=out_dtype, device=DEV)
        assert K.gemm_tc(dx, dw, out, bias=db, splits=splits)
        tol = dict(atol=1e-3, rtol=1e-3) if out_dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
        assert torch.allclose(out.float().cpu(), want, **tol)
    base = rnd((T, N), torch.float32, seed=24)
    acc = base.to(DEV).clone()
    assert K.gemm_tc(dx, dw, acc, bias=db, accumulate=True, splits=splits)
    assert torch.allclose(acc.cpu(), base + want, atol=2e-3, rtol=1e-3)
    gu = ref_product(x, w)
    gated = torch.full((T, N // 2), 7.0, dtype=BF, device=DEV)
    assert K.gemm_tc(dx, dw, gated, glu="silu", splits=splits)
    torch.cuda.synchronize()
    assert K.gemm_tc_status() == 0
    assert torch.allclose(gated.float().cpu(), P.silu(gu[:, 0::2]) * gu[:, 1::2], atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("kind", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("T,N,K_,splits", [(8, 512, 256, 0), (45, 352, 64, 0), (100, 400, 120, 0), (8, 1024, 2048, 4),
                                           (600, 3000, 512, 0)])
@pytest.mark.parametrize("bias_dtype", [None, BF, torch.float32])
def test_gemm_tc_gated(K, kind, T, N, K_, splits, bias_dtype):
    """act(gate + b_gate) * (up + b_up) with gate and up rows (and their biases) alternating."""
    x, w = rnd((T, K_), BF, seed=7), rnd((N, K_), BF, 0.05, seed=8)
    b = None if bias_dtype is None else rnd((N,), bias_dtype, 0.5, seed=9)
    gu = ref_product(x, w, b)
    g, u = gu[:, 0::2], gu[:, 1::2]
    want = (P.silu(g) if kind == "silu" else torch.nn.functional.gelu(g, approximate="tanh")) * u
    out = torch.full((T, N // 2), 7.0, dtype=BF, device=DEV)
    assert K.gemm_tc(x.to(DEV), w.to(DEV), out, bias=None if b is None else b.to(DEV), glu=kind, splits=splits)
    torch.cuda.synchronize()
    assert K.gemm_tc_status() == 0
    assert torch.allclose(out.float().cpu(), want, atol=3e-2, rtol=2e-2)


def test_gemm_tc_rows_of_wider_buffers_and_odd_output_stride(K):
    xb = rnd((20, 300), BF, seed=9).to(DEV)
    x = xb[:, 40:168]                                     # row stride 300 is no multiple of 8: refused
    w = rnd((50, 128), BF, 0.05, seed=10).to(DEV)
    out = torch.empty(20, 50, dtype=torch.float32, device=DEV)
    assert K.gemm_tc(x, w, out) is False
    xb = rnd((20, 304), BF, seed=9).to(DEV)
    x = xb[:, 40:168]
    assert K.gemm_tc(x, w, out) == 1                      # output rows of 50 floats: stored by the threads
    assert torch.allclose(out.cpu(), ref_product(x.cpu(), w.cpu()), atol=1e-3, rtol=1e-3)
    wide = torch.zeros(20, 64, dtype=torch.float32, device=DEV)
    assert K.gemm_tc(x, w, wide[:, :50], accumulate=True)  # output rows inside a wider buffer: through TMA
    assert torch.allclose(wide[:, :50].cpu(), ref_product(x.cpu(), w.cpu()), atol=1e-3, rtol=1e-3)
    assert (wide[:, 50:] == 0).all()
    assert K.gemm_tc_status() == 0
    with pytest.raises(K.KernelError):
        K.gemm_tc(x.float(), w, out)


# ------------------------------------------------------------------ attention
def run_decode(K, nh, nkv, hd, lens_past, window, n_splits, seed=20):
    lens_new = [1] * len(lens_past)
    ks, vs, q, positions, seq = dense_attention_case(BF, nh, nkv, hd, lens_past, lens_new, seed=seed)
    kp, vp, table = paged(ks, vs, 64, BF, seed=2)
    T = q.shape[0]
    out = torch.zeros(T, nh * hd, dtype=BF, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    wide = torch.zeros(T, nh * hd + 64, dtype=BF)
    wide[:, :nh * hd] = q.reshape(T, nh * hd)
    po = torch.empty(T * nh * n_splits * hd, device=DEV)
    pm = torch.empty(T * nh * n_splits * 2, device=DEV)
    assert K.attention_decode(wide.to(DEV), out, nh, nkv, hd, scale, window,
                              torch.tensor(positions, dtype=torch.int32, device=DEV),
                              torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV),
                              64, n_splits, po, pm)
    torch.cuda.synchronize()
    assert K.attention_tc_status() == 0
    want = plain_attention_rows(ks, vs, q, positions, seq, scale, window)
    return out.float().cpu().view(T, nh, hd), want


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (4, 4), (16, 1), (6, 3)])
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("n_splits", [1, 3, 8])
def test_attention_decode(K, hd, nh, nkv, window, n_splits):
    got, want = run_decode(K, nh, nkv, hd, [0, 130, 63, 300, 64], window, n_splits)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)


def run_decode_flat(K, nh, nkv, hd, lens_past, window, n_blocks, seed=20):
    lens_new = [1] * len(lens_past)
    ks, vs, q, positions, seq = dense_attention_case(BF, nh, nkv, hd, lens_past, lens_new, seed=seed)
    kp, vp, table = paged(ks, vs, 64, BF, seed=2)
    T = q.shape[0]
    out = torch.zeros(T, nh * hd, dtype=BF, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    wide = torch.zeros(T, nh * hd + 64, dtype=BF)
    wide[:, :nh * hd] = q.reshape(T, nh * hd)
    n_blocks = n_blocks or K.attention_decode_flat_blocks(T, nh, nkv, hd)
    assert n_blocks > 0
    # scratch full of NaN: whatever the merge reads must have been written by this call
    scratch = torch.full((K.attention_decode_flat_scratch(T, nh, nkv, hd, n_blocks),), float("nan"), device=DEV)
    counters = torch.zeros(T * nkv, dtype=torch.int32, device=DEV)
    args = (wide.to(DEV), out, nh, nkv, hd, scale, window, torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(seq, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64, n_blocks,
            counters, scratch)
    assert K.attention_decode_flat(*args)
    first = out.clone()
    assert K.attention_decode_flat(*args)            # the counters are back at zero: a second call is the same
    torch.cuda.synchronize()
    assert K.attention_tc_status() == 0
    assert int(counters.abs().sum()) == 0 and torch.equal(first, out)
    want = plain_attention_rows(ks, vs, q, positions, seq, scale, window)
    return out.float().cpu().view(T, nh, hd), want


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (4, 4), (16, 1), (6, 3)])
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("n_blocks", [0, 1, 5, 23])
def test_attention_decode_flat(K, hd, nh, nkv, window, n_blocks):
    """The flat kernel: blocks take equal runs of pages that start and end inside sequences.  0 blocks: one
    resident wave (more blocks than pages here: most have nothing to do); 1: one block walks every sequence;
    5 and 23: runs that straddle kv heads and sequences of unequal lengths."""
    got, want = run_decode_flat(K, nh, nkv, hd, [0, 130, 63, 300, 64, 1000, 5], window, n_blocks)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("n_blocks", [0, 3, 40])
def test_attention_decode_flat_many_short_sequences(K, hd, n_blocks):
    """The division among blocks counts an item's fixed work beside its pages: with many sequences of one or
    two pages and a few long ones, blocks begin and end in that fixed part, hold many whole items, or hold
    none of an item's pages; every page is still read once and every piece merged."""
    lens = [3, 70, 1, 64, 127, 0, 65, 9] * 12 + [900, 2, 2, 450]
    got, want = run_decode_flat(K, 8, 2, hd, lens, None, n_blocks, seed=31)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)


def test_attention_decode_flat_many_tokens(K):
    """More tokens than a warp scans at once, lengths of every residue."""
    lens = [(i * 37) % 200 for i in range(70)]
    got, want = run_decode_flat(K, 4, 2, 64, lens, None, 0, seed=21)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)
    got, want = run_decode_flat(K, 4, 2, 128, lens, 50, 7, seed=22)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hd,rot", [(64, 64), (128, 128), (128, 64), (64, 0)])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (6, 3)])
@pytest.mark.parametrize("store", [True, False])
@pytest.mark.parametrize("n_blocks,window", [(0, None), (5, None), (5, 100)])
def test_attention_decode_flat_with_rotation_and_cache_write(K, hd, rot, nh, nkv, store, n_blocks, window):
    """The flat kernel doing the step's rotation and cache write itself, against rope_store followed by the
    same kernel without them: the same output, the same rows in the cache, qkv left as it was.  Positions at
    the start, the end and the middle of a page; the cache row of the new token holds poison beforehand."""
    lens_past = [0, 130, 63, 300, 64, 1000, 5, 127]
    T = len(lens_past)
    ks = [rnd((p + 1, nkv, hd), BF, seed=50 + 10 * b) for b, p in enumerate(lens_past)]
    vs = [rnd((p + 1, nkv, hd), BF, seed=51 + 10 * b) for b, p in enumerate(lens_past)]
    kp, vp, table = paged(ks, vs, 64, BF, seed=4)
    for b, p in enumerate(lens_past):                       # the new token is not in the cache yet
        kp[table[b, p // 64], :, p % 64] = 777.0
        vp[table[b, p // 64], :, p % 64] = -777.0
    width = (nh + (2 * nkv if store else 0)) * hd
    qkv = rnd((T, width), BF, seed=60).to(DEV)
    inv = P.rope_inverse_frequencies(rot, 500000.0, None).to(device=DEV, dtype=torch.float32) if rot else None
    positions = torch.tensor(lens_past, dtype=torch.int32, device=DEV)
    seq = torch.arange(T, dtype=torch.int32, device=DEV)
    table = table.to(DEV)
    scale = 1.0 / math.sqrt(hd)
    nb = n_blocks or K.attention_decode_flat_blocks(T, nh, nkv, hd)

    def run(fused):
        k_pages, v_pages, rows = kp.to(DEV), vp.to(DEV), qkv.clone()
        if not store:                                       # somebody else has written the new rows already
            for b, p in enumerate(lens_past):
                k_pages[table[b, p // 64], :, p % 64] = ks[b][p].to(DEV)
                v_pages[table[b, p // 64], :, p % 64] = vs[b][p].to(DEV)
        out = torch.zeros(T, nh * hd, dtype=BF, device=DEV)
        scratch = torch.full((K.attention_decode_flat_scratch(T, nh, nkv, hd, nb),), float("nan"), device=DEV)
        counters = torch.zeros(T * nkv, dtype=torch.int32, device=DEV)
        if not fused:
            K.rope_store(rows, nh, nkv if store else 0, hd, rot, inv, positions, seq, table,
                         k_pages if store else None, v_pages if store else None, 64)
        assert K.attention_decode_flat(rows, out, nh, nkv, hd, scale, window, positions, seq, table, k_pages, v_pages,
                                       64, nb, counters, scratch, rope=(inv, rot, store) if fused else None)
        torch.cuda.synchronize()
        assert K.attention_tc_status() == 0 and int(counters.abs().sum()) == 0
        return out, k_pages, v_pages, rows

    out_f, k_f, v_f, rows_f = run(True)
    out_u, k_u, v_u, _ = run(False)
    assert torch.equal(rows_f, qkv)
    assert torch.equal(k_f, k_u) and torch.equal(v_f, v_u)
    assert torch.allclose(out_f.float(), out_u.float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("kernel", ["mma", "fmha"])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (4, 4), (16, 1)])
@pytest.mark.parametrize("window", [None, 37, 100])
def test_attention_prefill(K, kernel, hd, nh, nkv, window):
    """mma: the mma.sync kernel (64 query rows a block); fmha: the tcgen05 kernel (128 rows, accumulators in
    tensor memory).  Sequences shorter and longer than a tile, continued ones, one of a single token."""
    lens_past, lens_new = [0, 130, 63, 0, 5], [21, 1, 70, 300, 128]
    ks, vs, q, positions, seq = dense_attention_case(BF, nh, nkv, hd, lens_past, lens_new, seed=30)
    kp, vp, table = paged(ks, vs, 64, BF, seed=3)
    T = q.shape[0]
    out = torch.zeros(T, nh * hd, dtype=BF, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    cu = [0]
    for n in lens_new:
        cu.append(cu[-1] + n)
    fn = K.attention_prefill if kernel == "mma" else K.attention_prefill_fmha
    assert fn(q.reshape(T, nh * hd).to(DEV), out, len(lens_new), max(lens_new), nh, nkv, hd, scale,
              window, torch.tensor(cu, dtype=torch.int32, device=DEV),
              torch.tensor(lens_past, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV), vp.to(DEV), 64)
    torch.cuda.synchronize()
    assert K.attention_tc_status() == 0 and K.attention_fmha_status() == 0
    want = plain_attention_rows(ks, vs, q, positions, seq, scale, window)
    assert torch.allclose(out.float().cpu().view(T, nh, hd), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("kernel", ["decode", "flat", "prefill", "fmha"])
@pytest.mark.parametrize("hd", [64, 128])
def test_tc_attention_finds_one_far_key_and_respects_the_window_edge(K, kernel, hd):
    """One key is made to dominate: far back among hundreds (every page position, split boundary), then just
    inside and just outside the window.  The output must be that key's value, or must not be."""
    nh, nkv, n = 2, 1, 700
    scale = 1.0
    cases = [(far, None, True) for far in (0, 3, 63, 64, 389, 640, 699)]
    cases += [(n - 1 - 49, 50, True), (n - 1 - 50, 50, False)]
    for far, window, visible in cases:
        k = rnd((n, nkv, hd), BF, 0.1, seed=40)
        v = rnd((n, nkv, hd), BF, 1.0, seed=41)
        q = rnd((1, nh, hd), BF, 0.1, seed=42)
        k[far] = (q[0, 0].float() * 400.0).to(BF)
        kp, vp, table = paged([k], [v], 64, BF, seed=far)
        out = torch.zeros(1, nh * hd, dtype=BF, device=DEV)
        if kernel == "decode":
            ns = 4
            po = torch.empty(nh * ns * hd, device=DEV)
            pm = torch.empty(nh * ns * 2, device=DEV)
            assert K.attention_decode(q.reshape(1, -1).to(DEV), out, nh, nkv, hd, scale, window,
                                      torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                                      torch.zeros(1, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV),
                                      vp.to(DEV), 64, ns, po, pm)
        elif kernel == "flat":
            nb = 3
            scratch = torch.full((K.attention_decode_flat_scratch(1, nh, nkv, hd, nb),), float("nan"), device=DEV)
            assert K.attention_decode_flat(q.reshape(1, -1).to(DEV), out, nh, nkv, hd, scale, window,
                                           torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                                           torch.zeros(1, dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV),
                                           vp.to(DEV), 64, nb, torch.zeros(nkv, dtype=torch.int32, device=DEV),
                                           scratch)
        else:
            fn = K.attention_prefill if kernel == "prefill" else K.attention_prefill_fmha
            assert fn(q.reshape(1, -1).to(DEV), out, 1, 1, nh, nkv, hd, scale, window,
                                       torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                       torch.tensor([n - 1], dtype=torch.int32, device=DEV), table.to(DEV), kp.to(DEV),
                                       vp.to(DEV), 64)
        got = out.float().cpu().view(nh, hd)
        hit = torch.allclose(got[0], v[far, 0].float(), atol=3e-2)
        assert hit == visible, f"{kernel} hd={hd}: key {far}, window {window}"
        want = plain_attention_rows([k], [v], q, [n - 1], [0], scale, window)
        assert torch.allclose(got, want[0], atol=3e-2, rtol=2e-2)
    assert K.attention_tc_status() == 0


@pytest.mark.parametrize("library", ["gemm_tc", "attention_tc", "attention_fmha"])
def test_a_bounded_wait_that_runs_out_is_reported_and_the_library_goes_on(K, library):
    """The give-up path of the kernels' waits, run on purpose: a block waits (4096 polls) on a barrier in its own
    shared memory that nothing arrives on.  Nothing is in flight, nothing faults; the wait returns false, the
    library's error word holds code 90 once, and the next real call is right."""
    K.require((library,))
    status = {"gemm_tc": K.gemm_tc_status, "attention_tc": K.attention_tc_status,
              "attention_fmha": K.attention_fmha_status}[library]
    assert status() == 0
    passed, flag = K.wait_selftest(library, polls=4096)
    assert passed == 0 and flag == 1                     # the wait gave up and told the other warps of its block
    assert K.wait_errors()[library] == 90                # read through the call the engine uses ...
    assert status() == 0                                 # ... which cleared the word
    assert "on purpose" in K.describe_wait_errors({library: 90})
    # the library is as usable as before
    x = rnd((8, 256), BF, seed=1).to(DEV)
    w = rnd((384, 256), BF, 0.05, seed=2).to(DEV)
    out = torch.empty(8, 384, dtype=torch.float32, device=DEV)
    assert K.gemm_tc(x, w, out)
    assert torch.allclose(out.cpu(), ref_product(x.cpu(), w.cpu()), atol=1e-3, rtol=1e-3)
    got, want = run_decode(K, 8, 2, 64, [5, 130, 64], None, 2)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)
    assert all(c == 0 for c in K.wait_errors().values())
    with pytest.raises(K.KernelError):
        K.wait_selftest("elementwise")


def test_tc_attention_refuses_other_head_sizes(K):
    q = torch.zeros(1, 48, dtype=BF, device=DEV)
    out = torch.zeros(1, 48, dtype=BF, device=DEV)
    pages = torch.zeros(1, 1, 64, 48, dtype=BF, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    assert K.attention_prefill(q, out, 1, 1, 1, 1, 48, 1.0, None, z, z, z.view(1, 2), pages, pages, 64) is False


@pytest.mark.parametrize("T", [1, 8, 17, 41, 50, 64])
@pytest.mark.parametrize("d,k1,n2", [(256, 2048, 640), (4096, 512, 256), (200, 1024, 136), (256, 128, 64)])
@pytest.mark.parametrize("gain_dtype", [torch.float32, BF])
def test_gemm_tc_carries_an_rmsnorm_between_two_products(K, T, d, k1, n2, gain_dtype):
    """residual += a W1^T with the first half of the norm (x * gain as bf16, sums of squares per tile row), then
    (x * gain) W2^T scaled by 1 / sqrt(mean x^2 + eps) per row, plain and with the gated activation: the same
    as the residual sum, an RMSNorm kernel and the product."""
    eps = 1e-5
    a = rnd((T, k1), BF, 1.0, seed=1).to(DEV)
    w1 = rnd((d, k1), BF, 0.05, seed=2).to(DEV)
    x0 = rnd((T, d), torch.float32, 1.0, seed=3).to(DEV)
    gain = (1.0 + 0.2 * rnd((d,), torch.float32, 1.0, seed=4)).to(gain_dtype).to(DEV)
    w2 = rnd((n2, d), BF, 0.05, seed=5).to(DEV)
    bias = rnd((n2,), torch.float32, 1.0, seed=6).to(DEV)
    x = x0.clone()
    hb = torch.full((T, d), float("nan"), dtype=BF, device=DEV)
    ssq = torch.full((T, -(-d // 128)), float("nan"), device=DEV)
    done = K.gemm_tc(a, w1, x, accumulate=True, norm_out=(gain, 0.0, hb, ssq))
    x_ref = x0 + a.float() @ w1.float().t()
    assert torch.allclose(x, x_ref, atol=2e-3, rtol=2e-3)
    if done != 2:
        # too few K blocks to split over a cluster: the product says so and leaves hb and ssq alone
        assert done == 1 and torch.isnan(hb.float()).all() and torch.isnan(ssq).all()
        return
    assert torch.allclose(ssq.sum(1), (x * x).sum(1), rtol=1e-5)
    assert torch.equal(hb, (x * gain.float()).to(BF))
    h_ref = (x * (1.0 / torch.sqrt((x * x).mean(1, keepdim=True) + eps)) * gain.float()).to(BF)
    want = h_ref.float() @ w2.float().t() + bias
    got = torch.zeros(T, n2, device=DEV)
    assert K.gemm_tc(hb, w2, got, bias=bias, row_scale=(ssq, eps))
    torch.cuda.synchronize()
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 1e-2 * scale
    # the gated mode: rows of w2 alternate gate and up
    gu = h_ref.float() @ w2.float().t()
    want_act = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
    act = torch.zeros(T, n2 // 2, dtype=BF, device=DEV)
    assert K.gemm_tc(hb, w2, act, glu="silu", row_scale=(ssq, eps))
    torch.cuda.synchronize()
    assert (act.float() - want_act).abs().max().item() <= 2e-2 * max(want_act.abs().max().item(), 1e-3)
    assert K.gemm_tc_status() == 0
