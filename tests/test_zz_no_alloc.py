"""The decode attention entry point that allocates nothing (csrc/attention_noalloc.h), called through its
exported C symbol and compared with the regular entry point, whose scratch the caller allocates.

Some hosts of this library may not call cudaMalloc when they need attention (a frozen memory pool, a
runtime that owns all device memory); for them the library keeps the scratch of the key splits in a
device array of its own.  This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_long, c_void_p

import pytest
import torch

from test_gpu_kernels import DEV, dense_attention_case, paged, plain_attention_rows

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
SCRATCH_FLOATS = 2 * 1024 * 1024


def entry_points():
    from ziglm_b200.csrc import load
    lib = load("attention_tc")
    fn = lib.zlm_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p,
                   c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p]
    fn.restype = c_int
    msg = lib.zlm_attention_decode_noalloc_error
    msg.argtypes = [c_int]
    msg.restype = ctypes.c_char_p
    return fn, msg


def wait_status():
    """The error word of the entry point's own bounded waits (0: every wait completed), read and cleared."""
    from ziglm_b200.csrc import load
    status = load("attention_tc").zlm_attention_decode_noalloc_status
    status.argtypes = [ctypes.POINTER(c_int)]
    status.restype = c_int
    out = c_int(-7)
    assert status(ctypes.byref(out)) == 0
    return out.value


def case(nh, nkv, hd, lens_past, seed):
    ks, vs, q, positions, seq = dense_attention_case(BF, nh, nkv, hd, lens_past, [1] * len(lens_past), seed=seed)
    kp, vp, table = paged(ks, vs, 64, BF, seed=seed)
    T = q.shape[0]
    return dict(q=q.reshape(T, nh * hd).to(DEV), kp=kp.to(DEV), vp=vp.to(DEV), table=table.to(DEV),
                pos=torch.tensor(positions, dtype=torch.int32, device=DEV),
                seq=torch.tensor(seq, dtype=torch.int32, device=DEV), T=T,
                plain=(ks, vs, q, positions, seq))


def call_noalloc(fn, c, out, nh, nkv, hd, scale, window, n_splits):
    return fn(c["q"].data_ptr(), c["q"].stride(0), out.data_ptr(), c["T"], nh, nkv, hd, scale, window,
              c["pos"].data_ptr(), c["seq"].data_ptr(), c["table"].data_ptr(), c["table"].stride(0),
              c["kp"].data_ptr(), c["vp"].data_ptr(), c["kp"].shape[0], 64, n_splits,
              torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, 0), (6, 3, 64, 45)])
def test_no_alloc_entry_point_equals_the_regular_one_twice_in_a_row(nh, nkv, hd, window):
    from ziglm_b200 import kernels
    fn, msg = entry_points()
    scale = 1.0 / math.sqrt(hd)
    # Two different problems one after the other.  The first is large and fills much of the shared scratch; the
    # second has fewer rows and fewer splits, so every partial result it reads lies where the first call left
    # other values: a wrong offset into the array would read those.  The second also runs on a stream of its own.
    side = torch.cuda.Stream()
    for seed, lens_past, n_splits, stream in ((11, [0, 130, 63, 300, 64, 700, 5, 256], 12, None),
                                              (12, [500, 7, 129], 2, side)):
        c = case(nh, nkv, hd, lens_past, seed)
        T = c["T"]
        want = torch.zeros(T, nh * hd, dtype=BF, device=DEV)
        po = torch.empty(T * nh * n_splits * hd, device=DEV)
        pm = torch.empty(T * nh * n_splits * 2, device=DEV)
        assert kernels.attention_decode(c["q"], want, nh, nkv, hd, scale, window or None, c["pos"], c["seq"],
                                        c["table"], c["kp"], c["vp"], 64, n_splits, po, pm)
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream or torch.cuda.current_stream()):
            rc = call_noalloc(fn, c, got, nh, nkv, hd, scale, window, n_splits)
        assert rc == 0, msg(rc).decode()
        torch.cuda.synchronize()
        # against the plain statement of attention, not only against the other entry point
        plain = plain_attention_rows(*c["plain"], scale, window or None)
        assert torch.allclose(got.float().cpu().view(T, nh, hd), plain, atol=2e-2, rtol=2e-2)
        assert torch.equal(got, want)              # the same kernels on the same inputs
    assert wait_status() == 0


def test_no_alloc_entry_point_with_no_tokens_does_nothing():
    fn, msg = entry_points()
    c = case(4, 2, 64, [10, 20], 14)
    out = torch.full((2, 4 * 64), 3.0, dtype=BF, device=DEV)
    c0 = dict(c, T=0)
    assert call_noalloc(fn, c0, out, 4, 2, 64, 0.125, 0, 2) == 0
    torch.cuda.synchronize()
    assert (out == 3.0).all() and wait_status() == 0


def test_no_alloc_entry_point_refuses_what_exceeds_its_scratch():
    fn, msg = entry_points()
    nh, nkv, hd = 32, 8, 128
    c = case(nh, nkv, hd, [10] * 16, 13)
    out = torch.zeros(16, nh * hd, dtype=BF, device=DEV)
    n_splits = SCRATCH_FLOATS // (16 * nh * (hd + 2)) + 1
    rc = call_noalloc(fn, c, out, nh, nkv, hd, 0.1, 0, n_splits)
    assert rc == -3 and b"scratch" in msg(rc)
    assert (out == 0).all()                        # nothing was launched
    assert call_noalloc(fn, c, out, nh, nkv, hd, 0.1, 0, n_splits - 1) == 0
    torch.cuda.synchronize()
    assert call_noalloc(fn, c, out, nh, nkv, 48, 0.1, 0, 1) == -2
    assert wait_status() == 0
