"""Typed Python wrappers of the CUDA entry points in ``csrc/``.

Every wrapper checks what the kernel cannot (device, dtype, contiguity, sizes it
refuses), passes raw pointers and the current CUDA stream through the C ABI and
raises :class:`KernelError` on a non-zero status.  There is no CPU path: a call
with a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional, Tuple

import torch

from .csrc import builder as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_launches = 0   # kernels launched through these wrappers since the last reset


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


def launches() -> int:
    return _launches


def reset_launches() -> None:
    global _launches
    _launches = 0


def reset_launches_by(n: int) -> None:
    """Take back ``n`` counted launches (calls recorded into a CUDA graph launch nothing)."""
    global _launches
    _launches -= n


def code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


_PROTOTYPES = {
    "elementwise": {
        "zlm_embed": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "zlm_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_float,
                        c_void_p],
        "zlm_gated_act": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "zlm_add": [c_void_p, c_void_p, c_long, c_void_p],
        "zlm_convert": [c_void_p, c_int, c_void_p, c_int, c_long, c_void_p],
        "zlm_fill_normal": [c_void_p, c_int, c_long, ctypes.c_ulonglong, c_float, c_float, c_void_p],
    },
    "gemm_generic": {
        "zlm_gemm_generic": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_long, c_long, c_long, c_void_p],
    },
    "attention": {
        "zlm_rope_store": [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                           c_void_p, c_int, c_void_p, c_void_p, c_int, c_long, c_void_p],
        "zlm_attention_general": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_long, c_int,
                                  c_void_p, c_long, c_void_p],
        "zlm_attention_general_scratch": [c_int, c_int, c_int, c_int, c_int],
    },
    "attention_tc": {
        "zlm_attention_decode": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                 c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p],
        "zlm_attention_decode_flat": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                      c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p,
                                      c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p],
        "zlm_attention_decode_flat_blocks": [c_int, c_int, c_int, c_int],
        "zlm_attention_decode_flat_scratch": [c_int, c_int, c_int, c_int, c_int],
        "zlm_attention_prefill": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_void_p],
        "zlm_attention_tc_status": [c_void_p],
        "zlm_attention_tc_wait_selftest": [c_int, c_void_p, c_void_p],
    },
    "attention_fmha": {
        "zlm_attention_prefill_fmha": [c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                       c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int,
                                       c_void_p],
        "zlm_attention_fmha_status": [c_void_p],
        "zlm_attention_fmha_wait_selftest": [c_int, c_void_p, c_void_p],
    },
    "gemm_tc": {
        "zlm_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_long, c_long, c_long, c_int, c_void_p],
        "zlm_gemm_tc_norm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_long, c_long, c_long, c_int, c_void_p, c_int, c_float, c_void_p, c_long, c_void_p,
                             c_void_p, c_void_p, c_int, c_float, c_void_p],
        "zlm_gemm_tc_status": [c_void_p],
        "zlm_gemm_tc_wait_selftest": [c_int, c_void_p, c_void_p],
    },
    "sampling": {
        "zlm_sample_parts_scratch": [c_int],
        "zlm_sample_parts": [c_void_p, c_int, c_int, c_long, c_float, c_int, c_float, c_float, c_float, c_float, c_void_p,
                             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_void_p],
        "zlm_argmax": [c_void_p, c_int, c_int, c_long, c_void_p, c_void_p],
        "zlm_sample": [c_void_p, c_int, c_int, c_long, c_float, c_int, c_float, c_float, c_float, c_float, c_void_p,
                       c_int, c_void_p, c_void_p, c_void_p],
    },
}
_functions = {}


def _fn(library: str, name: str):
    f = _functions.get(name)
    if f is None:
        lib = _build.load(library)
        f = getattr(lib, name)
        f.argtypes = _PROTOTYPES[library][name]
        f.restype = c_long if name.endswith("_scratch") else c_int
        _functions[name] = f
    return f


def require(libraries) -> None:
    """Compile (if need be) and load the named kernel libraries, several at a time."""
    _build.build(list(libraries))
    for lib in libraries:
        _build.load(lib)


_STATUS = {-1: "bad argument", -2: "unsupported size or type", -3: "scratch memory too small"}


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: {_STATUS.get(status, 'error %d' % status)}")
    raise KernelError(f"{what}: CUDA error {status}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# The handle of the current stream of the current device.  torch.cuda.current_stream() builds a Stream object
# and resolves the device through several Python layers (a few microseconds a call, once per launch); the raw
# getter answers the same question in a fraction of that.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")


# ------------------------------------------------------------------ elementwise
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = float(table[tokens[t], :]) * scale;  out is float32 [T, d]."""
    _cuda(table, "table"); _cuda(tokens, "tokens", torch.int32); _cuda(out, "out", torch.float32)
    T, d = out.shape
    if table.shape[1] != d or tokens.numel() < T:
        raise KernelError("embed: shapes do not match")
    _check(_fn("elementwise", "zlm_embed")(table.data_ptr(), code(table.dtype), tokens.data_ptr(), out.data_ptr(),
                                           T, d, scale, _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None, weight_offset: float = 0.0) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * (weight + weight_offset); x is float32."""
    _cuda(x, "x", torch.float32); _cuda(weight, "weight"); _cuda(out, "out")
    n, d = out.shape
    if x.shape[1] != d or weight.numel() != d:
        raise KernelError("rmsnorm: shapes do not match")
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError("rmsnorm: fewer row indices than output rows")
    elif x.shape[0] < n:
        raise KernelError("rmsnorm: fewer input rows than output rows")
    _check(_fn("elementwise", "zlm_rmsnorm")(x.data_ptr(), weight.data_ptr(), code(weight.dtype), out.data_ptr(),
                                             code(out.dtype), _ptr(rows), n, d, eps, weight_offset, _stream()),
           "rmsnorm")


def gated_act(gu: torch.Tensor, out: torch.Tensor, activation: str = "silu", interleaved: bool = False) -> None:
    """out[t, j] = act(gate) * up for gu of shape [T, 2I]: gate j, up j in columns (j, I + j), or in columns
    (2j, 2j + 1) when ``interleaved``."""
    _cuda(gu, "gu"); _cuda(out, "out", gu.dtype)
    T, I = out.shape
    if gu.shape != (T, 2 * I):
        raise KernelError("gated_act: gu must be [T, 2*I]")
    kind = {"silu": 0, "gelu_tanh": 1}.get(activation)
    if kind is None:
        raise KernelError(f"gated_act: activation {activation!r} is not known (silu, gelu_tanh)")
    _check(_fn("elementwise", "zlm_gated_act")(gu.data_ptr(), out.data_ptr(), code(gu.dtype), T, I, kind,
                                               int(interleaved), _stream()), "gated_act")


def add_(y: torch.Tensor, x: torch.Tensor) -> None:
    _cuda(y, "y", torch.float32); _cuda(x, "x", torch.float32)
    if y.numel() != x.numel():
        raise KernelError("add_: sizes differ")
    _check(_fn("elementwise", "zlm_add")(y.data_ptr(), x.data_ptr(), y.numel(), _stream()), "add_")


def convert(src: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(src, "src"); _cuda(out, "out")
    if src.numel() != out.numel():
        raise KernelError("convert: sizes differ")
    _check(_fn("elementwise", "zlm_convert")(src.data_ptr(), code(src.dtype), out.data_ptr(), code(out.dtype),
                                             src.numel(), _stream()), "convert")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """out.flat[i] = mean + std * z(key, i) with z the counter-based standard normal value of
    ``ziglm_b200.weights.random_init.normal_values`` (the same bits on the device as there)."""
    _cuda(out, "out")
    _check(_fn("elementwise", "zlm_fill_normal")(out.data_ptr(), code(out.dtype), out.numel(),
                                                 int(key) & 0xFFFFFFFFFFFFFFFF, float(mean), float(std), _stream()),
           "fill_normal")


# ------------------------------------------------------------------------ gemm
def gemm_generic(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False) -> None:
    """out[M,N] (+)= x[M,K] @ w[N,K]^T (+ bias) on the CUDA cores; rows may be strided."""
    for t, n in ((x, "x"), (w, "w"), (out, "out")):
        if not t.is_cuda:
            raise KernelError(f"{n} must be on a CUDA device (there is no CPU path)")
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{n} must be a matrix with unit column stride")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes do not match: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulation needs a float32 output")
    if bias is not None:
        _cuda(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias length does not match")
    _check(_fn("gemm_generic", "zlm_gemm_generic")(
        x.data_ptr(), code(x.dtype), w.data_ptr(), code(w.dtype), _ptr(bias),
        code(bias.dtype) if bias is not None else F32, out.data_ptr(), code(out.dtype), int(accumulate),
        M, N, K, x.stride(0) if M > 1 else K, w.stride(0) if N > 1 else K, out.stride(0) if M > 1 else N,
        _stream()), "gemm_generic")


# ------------------------------------------------------------------- attention
def rope_store(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rotary_dim: int,
               inv_freq: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
               block_table: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
               page_size: int) -> None:
    """Rotate q and k of qkv[T, (n_heads+2 n_kv) head_dim] in place and store k, v in the cache pages.

    k_pages / v_pages: [n_pages, n_kv, page_size, head_dim] of one layer, or None to store nothing.
    block_table: int32 [B, stride]; row seq_of_token[t] lists the pages of token t's sequence.
    """
    _cuda(qkv, "qkv"); _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_store: qkv width does not match the head counts")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_store: the frequency table must hold rotary_dim/2 entries")
    page_stride = 0
    if k_pages is not None:
        _cuda(k_pages, "k_pages", qkv.dtype); _cuda(v_pages, "v_pages", qkv.dtype)
        if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelError("rope_store: cache pages must be [n_pages, n_kv, page_size, head_dim]")
        page_stride = k_pages.stride(0)
    _check(_fn("attention", "zlm_rope_store")(
        qkv.data_ptr(), code(qkv.dtype), qkv.stride(0), T, n_heads, n_kv, head_dim, rotary_dim, _ptr(inv_freq),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        _ptr(k_pages), _ptr(v_pages), page_size, page_stride, _stream()), "rope_store")


def attention_general_scratch(n_tokens: int, n_heads: int, n_kv: int, head_dim: int, max_keys: int) -> int:
    """Floats of scratch with which ``attention_general`` spreads a step of few tokens over more blocks (0: none
    is of use)."""
    return int(_fn("attention", "zlm_attention_general_scratch")(n_tokens, n_heads, n_kv, head_dim, max_keys))


def attention_general(qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                      window: Optional[int], positions: torch.Tensor, seq_of_token: torch.Tensor,
                      block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      page_size: int, max_keys: int = 0, scratch: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :] = softmax(q[t,h] . K[start..pos_t] * scale) @ V over the paged cache.

    The queries are the first n_heads*head_dim columns of each row of ``qkv`` (any row stride).
    ``max_keys`` (the most keys a token of the step sees) and ``scratch`` (float32, at least
    ``attention_general_scratch(...)`` elements) let a step of few tokens use more blocks; the result does not
    depend on them.
    """
    _cuda(out, "out", qkv.dtype); _cuda(k_pages, "k_pages", qkv.dtype); _cuda(v_pages, "v_pages", qkv.dtype)
    _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    if not qkv.is_cuda or qkv.stride(1) != 1:
        raise KernelError("attention: q must be on the device with unit column stride")
    T = out.shape[0]
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim:
        raise KernelError("attention: widths do not match the head counts")
    if head_dim % 8 or head_dim > 256:
        raise KernelError(f"attention: head size {head_dim} is not supported (a multiple of 8, at most 256)")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    _check(_fn("attention", "zlm_attention_general")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), code(qkv.dtype), T, n_heads, n_kv, head_dim, scale,
        int(window or 0), positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), page_size, k_pages.stride(0), int(max_keys),
        _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream()),
        "attention_general")
    if scratch is not None and max_keys > 0 and scratch.numel() >= attention_general_scratch(
            T, n_heads, n_kv, head_dim, max_keys) > 0:
        global _launches
        _launches += 1          # the fold of the parts is a second launch


def _tc_attention_ok(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_heads % n_kv == 0
            and n_heads // n_kv <= 16 and page_size == 64)


def attention_decode(qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                     window: Optional[int], positions: torch.Tensor, seq_of_token: torch.Tensor,
                     block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int,
                     n_splits: int, part_o: torch.Tensor, part_ml: torch.Tensor) -> bool:
    """Tensor-core attention for steps of one token per sequence (bf16, head size 64 or 128).

    Each token's query heads are grouped by key/value head so that the cache is read once per group; the keys
    of a sequence are split over ``n_splits`` blocks whose partial results go through the float32 scratch
    ``part_o`` [T*n_heads*n_splits*head_dim] and ``part_ml`` [T*n_heads*n_splits*2].  False if refused.
    """
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    _cuda(part_o, "part_o", torch.float32); _cuda(part_ml, "part_ml", torch.float32)
    T = out.shape[0]
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_decode: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim or qkv.shape[0] < T:
        raise KernelError("attention_decode: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_decode: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if part_o.numel() < T * n_heads * n_splits * head_dim or part_ml.numel() < T * n_heads * n_splits * 2:
        raise KernelError("attention_decode: the scratch is too small for this many splits")
    status = _fn("attention_tc", "zlm_attention_decode")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), T, n_heads, n_kv, head_dim, scale, int(window or 0),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, n_splits, part_o.data_ptr(),
        part_ml.data_ptr(), _stream())
    if status == -2:
        return False
    _check(status, "attention_decode")
    global _launches
    _launches += 1          # the merge of the splits is a second launch
    return True


def attention_decode_flat_blocks(n_tokens: int, n_heads: int, n_kv: int, head_dim: int) -> int:
    """Blocks of one resident wave of the flat decode kernel for a step of ``n_tokens`` (0: sizes it refuses)."""
    return int(_fn("attention_tc", "zlm_attention_decode_flat_blocks")(n_tokens, n_heads, n_kv, head_dim))


def attention_decode_flat_scratch(n_tokens: int, n_heads: int, n_kv: int, head_dim: int, n_blocks: int) -> int:
    """Floats of scratch the flat decode kernel needs with ``n_blocks`` blocks."""
    return int(_fn("attention_tc", "zlm_attention_decode_flat_scratch")(n_tokens, n_heads, n_kv, head_dim, n_blocks))


def attention_decode_flat(qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                          window: Optional[int], positions: torch.Tensor, seq_of_token: torch.Tensor,
                          block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int,
                          n_blocks: int, counters: torch.Tensor, scratch: torch.Tensor,
                          rope: Optional[Tuple[Optional[torch.Tensor], int, bool]] = None) -> bool:
    """Tensor-core attention for steps of one token per sequence, with the pages of all sequences of the
    step divided evenly over ``n_blocks`` blocks (one resident wave), whatever the sequences' lengths.  One
    launch: the block that finishes a sequence's last piece merges the pieces.

    ``scratch``: float32, at least ``attention_decode_flat_scratch(...)`` elements, any content.
    ``counters``: int32, one per (token, kv head), zero before the first call; a call that completes leaves
    them zero (a call that ended with a wait error does not: zero them again).  False if refused.

    ``rope`` = (inv_freq or None, rotary_dim, store): the kernel also does what ``rope_store`` does for the
    step's tokens, so that no kernel runs between the projection and the attention.  The rows of ``qkv`` are
    then [q heads | k heads | v heads] (k and v only with ``store``) as the projection left them; the query
    heads are rotated as they are loaded (``qkv`` itself is left alone) and, with ``store``, the new keys
    (rotated) and values go into the cache pages.  rotary_dim must be a multiple of 32.
    """
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32); _cuda(scratch, "scratch", torch.float32)
    _cuda(counters, "counters", torch.int32)
    T = out.shape[0]
    if counters.numel() < T * n_kv:
        raise KernelError("attention_decode_flat: one counter per (token, kv head) is needed")
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_decode_flat: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim or qkv.shape[0] < T:
        raise KernelError("attention_decode_flat: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_decode_flat: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if n_blocks <= 0:
        raise KernelError("attention_decode_flat: the number of blocks must be positive")
    fused, store, rot, inv_freq = 0, 0, 0, None
    if rope is not None:
        inv_freq, rot, store = rope
        fused = 1
        if inv_freq is None:
            rot = 0
        else:
            _cuda(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() * 2 != rot:
                raise KernelError("attention_decode_flat: the frequency table must hold rotary_dim/2 entries")
        if qkv.shape[1] < (n_heads + (2 * n_kv if store else 0)) * head_dim:
            raise KernelError("attention_decode_flat: the rows must hold the key and value heads to be stored")
    status = _fn("attention_tc", "zlm_attention_decode_flat")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), T, n_heads, n_kv, head_dim, scale, int(window or 0),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, n_blocks, counters.data_ptr(),
        scratch.data_ptr(), scratch.numel(), fused, int(bool(store)), int(rot), _ptr(inv_freq), _stream())
    if status == -2:
        return False
    if status == -1:
        raise KernelError("attention_decode_flat: bad arguments, or the scratch is too small for this many blocks")
    _check(status, "attention_decode_flat")
    return True


def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, n_seqs: int, max_new: int, n_heads: int, n_kv: int,
                      head_dim: int, scale: float, window: Optional[int], cu_seqlens: torch.Tensor,
                      past_lens: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                      v_pages: torch.Tensor, page_size: int) -> bool:
    """Tensor-core attention for prompt steps: sequence b brings tokens cu_seqlens[b]..cu_seqlens[b+1] of the
    packed stream after past_lens[b] cached ones (bf16, head size 64 or 128).  False if refused."""
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(past_lens, "past_lens", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_prefill: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim:
        raise KernelError("attention_prefill: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_prefill: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if cu_seqlens.numel() < n_seqs + 1 or past_lens.numel() < n_seqs:
        raise KernelError("attention_prefill: sequence arrays are too short")
    status = _fn("attention_tc", "zlm_attention_prefill")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), n_seqs, max_new, n_heads, n_kv, head_dim, scale,
        int(window or 0), cu_seqlens.data_ptr(), past_lens.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, _stream())
    if status == -2:
        return False
    _check(status, "attention_prefill")
    return True


def attention_prefill_fmha(qkv: torch.Tensor, out: torch.Tensor, n_seqs: int, max_new: int, n_heads: int, n_kv: int,
                           head_dim: int, scale: float, window: Optional[int], cu_seqlens: torch.Tensor,
                           past_lens: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, page_size: int) -> bool:
    """Prompt attention on the tcgen05 tensor cores (tiles of 128 queries, accumulators in tensor memory); same
    arguments as :func:`attention_prefill`.  False if refused."""
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(past_lens, "past_lens", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_prefill_fmha: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim:
        raise KernelError("attention_prefill_fmha: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_prefill_fmha: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if cu_seqlens.numel() < n_seqs + 1 or past_lens.numel() < n_seqs:
        raise KernelError("attention_prefill_fmha: sequence arrays are too short")
    status = _fn("attention_fmha", "zlm_attention_prefill_fmha")(
        qkv.data_ptr(), qkv.stride(0), qkv.shape[0], out.data_ptr(), n_seqs, max_new, n_heads, n_kv, head_dim, scale,
        int(window or 0), cu_seqlens.data_ptr(), past_lens.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, _stream())
    if status == -2:
        return False
    _check(status, "attention_prefill_fmha")
    return True


def attention_fmha_status() -> int:
    """0, or the code of a bounded wait that ran out inside the tcgen05 attention kernel (21 queries, 22 page,
    23 scores, 24 probabilities, 25 output, 26 stage never drained, 4 copies still in flight)."""
    out = ctypes.c_int(0)
    rc = _fn("attention_fmha", "zlm_attention_fmha_status")(ctypes.byref(out))
    if rc != 0:
        raise KernelError(f"attention_fmha_status: CUDA error {rc}")
    return out.value


def attention_tc_status() -> int:
    """0, or the code of a bounded wait that ran out inside a tensor-core attention kernel (11 a page never
    landed, 12 a stage never drained, 4 copies still in flight).  Synchronises the device."""
    out = ctypes.c_int(0)
    rc = _fn("attention_tc", "zlm_attention_tc_status")(ctypes.byref(out))
    if rc != 0:
        raise KernelError(f"attention_tc_status: CUDA error {rc}")
    return out.value


def decode_splits(n_tokens: int, n_kv: int, max_total: int, page_size: int = 64) -> int:
    """How many blocks share the keys of one sequence in a decode step: enough for two blocks per SM."""
    pages = max(1, -(-max_total // page_size))
    want = -(-296 // max(1, n_tokens * n_kv))
    return max(1, min(want, pages, 64))


def attention_with_rope(step, qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                        scale: float, window: Optional[int], io, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                        store: bool) -> bool:
    """Decode steps on the tensor-core path: rotation, cache write and attention in one kernel.  False when
    the step is not of that kind; the caller then runs ``rope_store`` and ``attention``."""
    if not (step.single_token and _tc_attention_ok(qkv.dtype, n_heads, n_kv, head_dim, io.page_size)):
        return False
    if inv_freq is not None and rotary_dim % 32:
        return False
    n_blocks = attention_decode_flat_blocks(step.n_tokens, n_heads, n_kv, head_dim)
    if n_blocks <= 0:
        return False
    need = attention_decode_flat_scratch(step.n_tokens, n_heads, n_kv, head_dim, n_blocks)
    scratch = step.ws.buf("attn_flat_scratch", (need,), torch.float32)
    counters = step.ws.buf("attn_flat_counters", (step.n_tokens * n_kv,), torch.int32, zeros=True)
    return attention_decode_flat(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions, step.seq_of_token,
                                 io.block_table, io.k_pages, io.v_pages, io.page_size, n_blocks, counters, scratch,
                                 rope=(inv_freq, rotary_dim, store))


def attention(step, qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
              window: Optional[int], io) -> None:
    """Attention of a step's tokens over the cache of the running layer; picks the kernel."""
    if _tc_attention_ok(qkv.dtype, n_heads, n_kv, head_dim, io.page_size):
        n_blocks = attention_decode_flat_blocks(step.n_tokens, n_heads, n_kv, head_dim) if step.single_token else 0
        if n_blocks > 0:
            need = attention_decode_flat_scratch(step.n_tokens, n_heads, n_kv, head_dim, n_blocks)
            scratch = step.ws.buf("attn_flat_scratch", (need,), torch.float32)
            counters = step.ws.buf("attn_flat_counters", (step.n_tokens * n_kv,), torch.int32, zeros=True)
            if attention_decode_flat(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions,
                                     step.seq_of_token, io.block_table, io.k_pages, io.v_pages, io.page_size,
                                     n_blocks, counters, scratch):
                return
        if step.single_token:
            n_splits = decode_splits(step.n_tokens, n_kv, step.max_total, io.page_size)
            part_o = step.ws.buf("attn_part_o", (step.n_tokens * n_heads * n_splits * head_dim,), torch.float32)
            part_ml = step.ws.buf("attn_part_ml", (step.n_tokens * n_heads * n_splits * 2,), torch.float32)
            if attention_decode(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions,
                                step.seq_of_token, io.block_table, io.k_pages, io.v_pages, io.page_size, n_splits,
                                part_o, part_ml):
                return
        else:
            # prompts: the tcgen05 kernel (tiles of 128 queries); a handful of tokens: the 64-row mma.sync one
            args = (qkv, out, step.n_seqs, step.max_new, n_heads, n_kv, head_dim, scale, window, step.cu_seqlens,
                    step.past_lens, io.block_table, io.k_pages, io.v_pages, io.page_size)
            if step.max_new >= 16 and attention_prefill_fmha(*args):
                return
            if attention_prefill(*args):
                return
    max_keys = min(step.max_total, window) if window else step.max_total
    need = attention_general_scratch(step.n_tokens, n_heads, n_kv, head_dim, max_keys)
    scratch = step.ws.buf("attn_parts", (need,), torch.float32) if need > 0 else None
    attention_general(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions, step.seq_of_token,
                      io.block_table, io.k_pages, io.v_pages, io.page_size, max_keys, scratch)


def fast_attention_libraries(dtype: torch.dtype, head_dim: int, n_heads: int = 1, n_kv: int = 1):
    """The sources of the tensor-core attention kernels if they take this shape, else nothing (the plain kernel runs)."""
    return ("attention_tc", "attention_fmha") if _tc_attention_ok(dtype, n_heads, n_kv, head_dim, 64) else ()


def fast_gemm_libraries():
    return ("gemm_tc",)


GLU_KINDS = {"silu": 1, "gelu_tanh": 2}


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, splits: int = 0, glu: Optional[str] = None, norm_out=None, row_scale=None):
    """out[T,N] (+)= x[T,K] @ w[N,K]^T (+ bias) on the tcgen05 tensor cores, bf16 operands.

    With ``glu`` ("silu" or "gelu_tanh") the rows of w (and the entries of bias) alternate gate and up rows and
    out is bf16 [T, N/2] holding act(gate + bias) * (up + bias).

    An RMSNorm between two products of a step of few tokens can ride on them.  ``norm_out`` = (gain, offset, hb,
    ssq) on the product before it (``accumulate`` into the float32 residual): it also leaves bf16(x * (gain +
    offset)) in ``hb`` [T, N] and sums of x^2 per tile row of 128 features in ``ssq`` [T, ceil(N/128)] (float32);
    the result is then 2 if it did and 1 if the launch it chose cannot (nothing is written to hb and ssq).
    ``row_scale`` = (ssq, eps) on the product after it, whose x is that ``hb``: every output row t is multiplied
    by 1 / sqrt(sum(ssq[t]) / K + eps) before the bias.

    Returns False, having done nothing, if the operands are not what TMA can read (a row stride that is no
    multiple of 8 elements, a base address off a 16-byte boundary); else a true value.
    """
    for t, n in ((x, "x"), (w, "w"), (out, "out")):
        if not t.is_cuda:
            raise KernelError(f"{n} must be on a CUDA device (there is no CPU path)")
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{n} must be a matrix with unit column stride")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: x and w must be bfloat16")
    T, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if glu else N
    if glu and (glu not in GLU_KINDS or N % 2 or out.dtype != torch.bfloat16):
        raise KernelError("gemm_tc: the gated mode needs silu or gelu_tanh, an even row count and a bf16 output")
    if w.shape[1] != K or out.shape != (T, n_out):
        raise KernelError(f"gemm: shapes do not match: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulation needs a float32 output")
    if bias is not None:
        _cuda(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias length does not match")
    gain = hb = ssq_out = ssq_in = None
    offset, eps, scale_p = 0.0, 0.0, 0
    fused = ctypes.c_int(0)
    if norm_out is not None:
        gain, offset, hb, ssq_out = norm_out
        _cuda(gain, "gain"); _cuda(hb, "hb", torch.bfloat16); _cuda(ssq_out, "ssq", torch.float32)
        if not accumulate or glu or gain.numel() != N or hb.shape != (T, N) or hb.stride(1) != 1 \
                or ssq_out.numel() < T * (-(-N // 128)) or gain.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_tc: norm_out needs accumulate, a gain of N elements, hb [T, N] and ssq [T, ceil(N/128)]")
    if row_scale is not None:
        ssq_in, eps = row_scale
        _cuda(ssq_in, "ssq", torch.float32)
        if T > 64 or ssq_in.dim() != 2 or ssq_in.shape[0] < T or not ssq_in.is_contiguous():
            raise KernelError("gemm_tc: row_scale needs at most 64 rows and ssq [T, P] contiguous")
        scale_p = ssq_in.shape[1]
    status = _fn("gemm_tc", "zlm_gemm_tc_norm")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), code(bias.dtype) if bias is not None else F32, out.data_ptr(),
        code(out.dtype), int(accumulate), GLU_KINDS[glu] if glu else 0, T, N, K, x.stride(0) if T > 1 else K,
        w.stride(0) if N > 1 else K, out.stride(0) if T > 1 else n_out, int(splits),
        _ptr(gain), code(gain.dtype) if gain is not None else F32, float(offset), _ptr(hb),
        hb.stride(0) if hb is not None and T > 1 else N, _ptr(ssq_out), ctypes.byref(fused), _ptr(ssq_in), scale_p,
        float(eps), _stream())
    if status == -2:
        return False
    _check(status, "gemm_tc")
    return 2 if fused.value else 1


def gemm_tc_status() -> int:
    """0, or the code of a bounded wait that ran out inside a tensor-core kernel since the last call
    (1 tile never landed, 2 stage never drained, 3 accumulator never completed, 4 copies still in flight).
    Synchronises the device."""
    out = ctypes.c_int(0)
    rc = _fn("gemm_tc", "zlm_gemm_tc_status")(ctypes.byref(out))
    if rc != 0:
        raise KernelError(f"gemm_tc_status: CUDA error {rc}")
    return out.value


WAIT_ERROR_NAMES = {
    1: "a tile never landed", 2: "a stage never drained", 3: "an accumulator never completed",
    4: "copies were still in flight when a block gave up", 11: "a cache page never landed",
    12: "a stage never drained", 21: "the queries never landed", 22: "a cache page never landed",
    23: "the scores never completed", 24: "the probabilities were never consumed", 25: "the output never completed",
    26: "a stage never drained", 27: "a tile address was off its boundary", 90: "a wait ran out on purpose (self-test)",
}


def wait_errors() -> dict:
    """The error words of the bounded waits of every tensor-core library this process has loaded: library name
    -> code (0: none).  Reading a word clears it.  Synchronises the device."""
    out = {}
    for lib, read in (("gemm_tc", gemm_tc_status), ("attention_tc", attention_tc_status),
                      ("attention_fmha", attention_fmha_status)):
        if _build.is_loaded(lib):
            out[lib] = read()
    return out


def wait_selftest(library: str, polls: int = 4096) -> Tuple[int, int]:
    """Run the give-up path of the bounded waits of ``library`` ("gemm_tc", "attention_tc" or "attention_fmha")
    once, on purpose and harmlessly: one block waits, with a limit of ``polls`` polls, on a barrier in its own
    shared memory that nothing arrives on (no copy, no tensor memory, nothing in flight), records code 90 in
    the library's error word and returns.  Result: (what the wait returned: 0 = gave up, the abort flag it
    left).  The library's status call then reports 90 once."""
    if library not in ("gemm_tc", "attention_tc", "attention_fmha"):
        raise KernelError(f"no bounded waits in {library!r}")
    seen = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    _check(_fn(library, f"zlm_{library}_wait_selftest")(int(polls), seen.data_ptr(), _stream()), "wait_selftest")
    torch.cuda.current_stream().synchronize()
    passed, flag = seen.tolist()
    return int(passed), int(flag)


def describe_wait_errors(codes: dict) -> str:
    return "; ".join(f"{lib}: code {c} ({WAIT_ERROR_NAMES.get(c, 'unknown')})" for lib, c in codes.items() if c)


def fast_gemm(linear, x: torch.Tensor, out: torch.Tensor, accumulate: bool, norm_out=None, row_scale=None):
    """Run the product on the tensor-core kernels if they take it (see ``gemm_tc`` for the result); False if
    they do not."""
    if x.dtype != torch.bfloat16 or linear.weight.dtype != torch.bfloat16:
        return False
    if out.dtype not in (torch.float32, torch.bfloat16):
        return False
    return gemm_tc(x, linear.weight, out, bias=linear.bias, accumulate=accumulate, norm_out=norm_out,
                   row_scale=row_scale)


# -------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = the id of the largest logit of row r (lowest id on ties)."""
    _cuda(out, "out", torch.int32)
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be a float32 matrix on the device with unit column stride")
    rows, V = logits.shape
    if out.numel() < rows:
        raise KernelError("argmax: the output is too short")
    _check(_fn("sampling", "zlm_argmax")(logits.data_ptr(), rows, V, logits.stride(0) if rows > 1 else V,
                                         out.data_ptr(), _stream()), "argmax")


def sample(logits: torch.Tensor, out: torch.Tensor, rng: torch.Tensor, temperature: float, top_k: int = 0,
           top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0, presence_penalty: float = 0.0,
           history: Optional[torch.Tensor] = None) -> None:
    """Draw one id per row.  rng: int64 [rows, 2] of (seed, counter).  history: int32 [rows, window], -1 = empty.

    The logits are changed in place when a penalty is on.
    """
    _cuda(out, "out", torch.int32); _cuda(rng, "rng", torch.int64)
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a float32 matrix on the device with unit column stride")
    rows, V = logits.shape
    if out.numel() < rows or rng.numel() < 2 * rows:
        raise KernelError("sample: output or rng too short")
    if not temperature > 0:
        raise KernelError("sample: the temperature must be positive (use argmax for greedy)")
    if top_k > 1024:
        raise KernelError("sample: top_k above 1024 is not supported")
    window = 0
    if history is not None:
        _cuda(history, "history", torch.int32)
        window = history.shape[1]
        if history.shape[0] < rows or window > 1024:
            raise KernelError("sample: history must be [rows, window] with window <= 1024")
    if 1 <= top_k <= 64 and window <= 256:
        # many blocks per row: each finds the k best of its slice, the last one to arrive cuts and draws
        counters, scratch = _sample_scratch(logits.device, rows)
        status = _fn("sampling", "zlm_sample_parts")(
            logits.data_ptr(), rows, V, logits.stride(0) if rows > 1 else V, temperature, int(top_k), top_p, min_p,
            repetition_penalty, presence_penalty, _ptr(history), window, rng.data_ptr(), out.data_ptr(),
            counters.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream())
        if status != -2:
            _check(status, "sample")
            return
    _check(_fn("sampling", "zlm_sample")(
        logits.data_ptr(), rows, V, logits.stride(0) if rows > 1 else V, temperature, int(top_k), top_p, min_p,
        repetition_penalty, presence_penalty, _ptr(history), window, rng.data_ptr(), out.data_ptr(), _stream()),
        "sample")


_SAMPLE_SCRATCH = {}


def _sample_scratch(device: torch.device, rows: int):
    """Counters and scratch of the many-block sampler, kept per device and grown as needed.  The counters (one
    per row, a buffer of their own so that their place does not move with the number of rows) start at zero
    and every call leaves them zero."""
    counters, scratch = _SAMPLE_SCRATCH.get(device, (None, None))
    need = int(_fn("sampling", "zlm_sample_parts_scratch")(rows))
    if counters is None or counters.numel() < rows:
        counters = torch.zeros(max(rows, 64), dtype=torch.int32, device=device)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 1), dtype=torch.float32, device=device)
    _SAMPLE_SCRATCH[device] = (counters, scratch)
    return counters, scratch
