"""ctypes front-end for the CPU oracle (``libratchet_oracle.so``).

TEST INFRASTRUCTURE, NOT PRODUCT CODE: only the tests, the smoke check and the CPU-baseline leg
of the benchmark import this module.  It restates ratchet-core's CPU device
(crates/ratchet-core/src/cpu/*.rs, crates/ratchet-core/src/quant.rs); see the header of
``ratchet_oracle.cpp`` for the parity status (floating point: parity unpinned at bit level).

All functions take and return numpy arrays.  f16 is ``np.float16``; bf16 is carried as
``np.uint16`` bit patterns with ``dt="bf16"``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libratchet_oracle.so")

F32, F16, BF16, I32, U32 = 0, 1, 2, 3, 4
_NP2DT = {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.int32): I32, np.dtype(np.uint32): U32}

BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3}
UNARY_OPS = {"gelu": 0, "tanh": 1, "exp": 2, "log": 3, "sin": 4, "cos": 5, "abs": 6, "sqrt": 7, "relu": 8,
             "floor": 9, "ceil": 10, "neg": 11, "silu": 12, "sigmoid": 13}


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the library is missing or stale."""
    src = os.path.join(_HERE, "ratchet_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libratchet_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_q8_nbytes.restype = C.c_uint64
        _lib.orc_q8_nbytes.argtypes = [C.c_uint64, C.c_int]
        _lib.orc_q8_scale_offset.restype = C.c_uint64
        _lib.orc_q8_scale_offset.argtypes = [C.c_uint64]
        _lib.orc_q4abs_nbytes.restype = C.c_uint64
        _lib.orc_q4abs_nbytes.argtypes = [C.c_uint64, C.c_int]
        _lib.orc_q4k_nbytes.restype = C.c_uint64
        _lib.orc_q4k_nbytes.argtypes = [C.c_uint64, C.c_int]
        for name in ("orc_quantize_q8", "orc_quantize_q4abs", "orc_quantize_q4k"):
            getattr(_lib, name).restype = C.c_uint64
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _dt(a: np.ndarray, dt=None) -> int:
    if dt == "bf16":
        return BF16
    return _NP2DT[a.dtype]


def _i64(seq):
    return (C.c_int64 * len(seq))(*[int(s) for s in seq])


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


# ----------------------------------------------------------------------------- quantisation
def q8_nbytes(numel: int, half: bool) -> int:
    return lib().orc_q8_nbytes(numel, int(half))


def q8_scale_offset(numel: int) -> int:
    return lib().orc_q8_scale_offset(numel)


def quantize_q8(x: np.ndarray) -> np.ndarray:
    """quant.rs:51-99. f32 input -> Q8_0F buffer, f16 input -> Q8_0H buffer (uint8 array)."""
    x = np.ascontiguousarray(x)
    half = x.dtype == np.float16
    assert half or x.dtype == np.float32
    out = np.zeros(q8_nbytes(x.size, half), np.uint8)
    n = lib().orc_quantize_q8(_p(x), C.c_uint64(x.size), int(half), _p(out))
    assert n == out.size
    return out


def dequantize_q8(buf: np.ndarray, shape, half: bool) -> np.ndarray:
    """quant.rs:101-164."""
    n = int(np.prod(shape))
    out = np.empty(n, np.float16 if half else np.float32)
    lib().orc_dequantize_q8(_p(buf), C.c_uint64(n), int(half), _p(out))
    return out.reshape(shape)


def quantize_q4abs(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x)
    half = x.dtype == np.float16
    out = np.zeros(lib().orc_q4abs_nbytes(x.size, int(half)), np.uint8)
    lib().orc_quantize_q4abs(_p(x), C.c_uint64(x.size), int(half), _p(out))
    return out


def dequantize_q4abs(buf: np.ndarray, shape, half: bool) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, np.float16 if half else np.float32)
    lib().orc_dequantize_q4abs(_p(buf), C.c_uint64(n), int(half), _p(out))
    return out.reshape(shape)


def q4k_nbytes(numel: int, half: bool) -> int:
    return lib().orc_q4k_nbytes(numel, int(half))


def q4k_offsets(numel: int, half: bool):
    off = (C.c_uint64 * 4)()
    lib().orc_q4k_offsets(C.c_uint64(numel), int(half), off)
    return list(off)


def quantize_q4k(x: np.ndarray, half: bool) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros(q4k_nbytes(x.size, half), np.uint8)
    lib().orc_quantize_q4k(_p(x), C.c_uint64(x.size), int(half), _p(out))
    return out


def dequantize_q4k(buf: np.ndarray, shape, half: bool) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, np.float16 if half else np.float32)
    lib().orc_dequantize_q4k(_p(buf), C.c_uint64(n), int(half), _p(out))
    return out.reshape(shape)


# ----------------------------------------------------------------------------- matmul
def matmul(lhs, rhs, bias=None, trans_lhs=False, trans_rhs=False, trans_dst=False, dt=None):
    """ops/matmul/mod.rs:392-466 + cpu/gemm.rs:59-127 (+ explicit bias add)."""
    lhs = np.ascontiguousarray(lhs)
    rhs = np.ascontiguousarray(rhs)
    assert lhs.dtype == rhs.dtype
    # upper bound of the output size: stacks * m * n
    ls, rs = list(lhs.shape), list(rhs.shape)
    rank = max(len(ls), len(rs))
    lsp = [1] * (rank - len(ls)) + ls
    rsp = [1] * (rank - len(rs)) + rs
    pre = [max(a, b) for a, b in zip(lsp[:-2], rsp[:-2])]
    m = lsp[-1] if trans_lhs else lsp[-2]
    n = rsp[-2] if trans_rhs else rsp[-1]
    out = np.empty(int(np.prod(pre, dtype=np.int64)) * m * n, lhs.dtype)
    dshape = (C.c_int64 * 8)()
    drank = C.c_int(0)
    if bias is not None:
        bias = np.ascontiguousarray(bias, lhs.dtype)
    rc = lib().orc_matmul(_dt(lhs, dt), _p(lhs), _i64(ls), len(ls), _p(rhs), _i64(rs), len(rs), _p(bias),
                          int(trans_lhs), int(trans_rhs), int(trans_dst), _p(out), dshape, C.byref(drank))
    if rc != 0:
        raise ValueError(f"oracle matmul rejected the shapes (code {rc})")
    return out.reshape([dshape[i] for i in range(drank.value)])


def gemv_q8(wbuf, N, K, half, x, bias=None, rows=None):
    """dequantize -> matmul for W[N,K] and x[K] without materialising W (CPU baseline helper)."""
    x = np.ascontiguousarray(x)
    y = np.zeros(N, x.dtype)
    r0, r1 = rows if rows is not None else (0, N)
    lib().orc_gemv_q8(_p(wbuf), C.c_uint64(N), C.c_uint64(K), int(half), _p(x), _dt(x), _p(bias), _p(y),
                      C.c_uint64(r0), C.c_uint64(r1))
    return y


# ----------------------------------------------------------------------------- elementwise
def binary(op: str, a, b, dt=None):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    out = np.empty_like(a)
    assert lib().orc_binary(_dt(a, dt), BINARY_OPS[op], _p(a), _p(b), _p(out), C.c_uint64(a.size)) == 0
    return out


def unary(op: str, x, dt=None):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    assert lib().orc_unary(_dt(x, dt), UNARY_OPS[op], _p(x), _p(out), C.c_uint64(x.size)) == 0
    return out


_DT2NP = {F32: np.float32, F16: np.float16, BF16: np.uint16, I32: np.int32, U32: np.uint32}


def cast(x, src_dt: int, dst_dt: int):
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, _DT2NP[dst_dt])
    assert lib().orc_cast(src_dt, dst_dt, _p(x), _p(out), C.c_uint64(x.size)) == 0
    return out


def layer_norm(x, scale, bias, eps, dt=None):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    N = x.shape[-1]
    assert lib().orc_layer_norm(_dt(x, dt), _p(x), _p(np.ascontiguousarray(scale)),
                                _p(None if bias is None else np.ascontiguousarray(bias)), C.c_float(eps), _p(out),
                                C.c_uint64(x.size // N), C.c_uint64(N)) == 0
    return out


def rms_norm(x, scale, eps, dt=None):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    N = x.shape[-1]
    assert lib().orc_rms_norm(_dt(x, dt), _p(x), _p(np.ascontiguousarray(scale)), C.c_float(eps), _p(out),
                              C.c_uint64(x.size // N), C.c_uint64(N)) == 0
    return out


def softmax(x, dim, dt=None):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    assert lib().orc_softmax(_dt(x, dt), _p(x), _p(out), C.c_uint64(x.size), C.c_uint64(x.shape[dim])) == 0
    return out


def rope(x, dim, base, offset):
    x = np.ascontiguousarray(x, np.float32)
    B, H, S, D = x.shape
    out = np.empty_like(x)
    lib().orc_rope(_p(x), _p(out), C.c_uint64(B), C.c_uint64(H), C.c_uint64(S), C.c_uint64(D), C.c_uint64(dim),
                   C.c_float(base), C.c_uint64(offset))
    return out


# ----------------------------------------------------------------------------- indexing / copies
def concat(inputs, dim):
    inputs = [np.ascontiguousarray(a) for a in inputs]
    rank = inputs[0].ndim
    shapes = []
    for a in inputs:
        shapes += list(a.shape)
    dshape = list(inputs[0].shape)
    dshape[dim] = sum(a.shape[dim] for a in inputs)
    out = np.empty(dshape, inputs[0].dtype)
    ptrs = (C.c_void_p * len(inputs))(*[a.ctypes.data for a in inputs])
    lib().orc_concat(ptrs, _i64(shapes), len(inputs), rank, dim, _p(out), inputs[0].itemsize)
    return out


def index_select(src, ids, dim):
    src = np.ascontiguousarray(src)
    ids = np.ascontiguousarray(ids, np.int32)
    dshape = list(src.shape)
    dshape[dim] = ids.size
    out = np.empty(dshape, src.dtype)
    lib().orc_index_select(_p(src), _i64(src.shape), src.ndim, _p(ids), C.c_uint64(ids.size), dim, _p(out), src.itemsize)
    return out


def index_select_q8(wbuf, shape, half, ids, dim):
    ids = np.ascontiguousarray(ids, np.int32)
    dshape = list(shape)
    dshape[dim] = ids.size
    out = np.empty(dshape, np.float16 if half else np.float32)
    lib().orc_index_select_q8(_p(wbuf), _i64(shape), int(half), _p(ids), C.c_uint64(ids.size), dim, _p(out))
    return out


def permute(src, perm):
    src = np.ascontiguousarray(src)
    out = np.empty([src.shape[p] for p in perm], src.dtype)
    assert lib().orc_permute(src.itemsize, _p(src), _i64(src.shape), src.ndim, (C.c_int * len(perm))(*perm), _p(out)) == 0
    return out


def slice_(src, ranges):
    src = np.ascontiguousarray(src)
    start = [r[0] for r in ranges]
    stop = [r[1] for r in ranges]
    out = np.empty([b - a for a, b in ranges], src.dtype)
    assert lib().orc_slice(src.itemsize, _p(src), _i64(src.shape), src.ndim, _i64(start), _i64(stop), _p(out)) == 0
    return out


def broadcast(src, to_shape, vector_fast_path=False):
    src = np.ascontiguousarray(src)
    out = np.empty(to_shape, src.dtype)
    assert lib().orc_broadcast(src.itemsize, _p(src), _i64(src.shape), src.ndim, _i64(to_shape), len(to_shape), _p(out),
                               int(vector_fast_path)) == 0
    return out


def cache(cache_arr, src, dim, offset):
    """Returns dst; ``cache_arr`` is updated in place (ops/cache.rs:73-103)."""
    assert cache_arr.flags.c_contiguous
    src = np.ascontiguousarray(src)
    dshape = list(cache_arr.shape)
    dshape[dim] = offset + src.shape[dim]
    out = np.empty(dshape, cache_arr.dtype)
    lib().orc_cache(_p(cache_arr), _i64(cache_arr.shape), _p(src), _i64(src.shape), cache_arr.ndim, dim, C.c_uint64(offset),
                    _p(out), cache_arr.itemsize)
    return out


def index_write(dst, src, start):
    assert dst.flags.c_contiguous
    src = np.ascontiguousarray(src)
    lib().orc_index_write(_p(dst), _i64(dst.shape), _p(src), _i64(src.shape), dst.ndim, _i64(start), dst.itemsize)
    return dst


def conv1d_k3(x, w, b, stride, pad):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    b = None if b is None else np.ascontiguousarray(b, np.float32)
    B, Cin, Lin = x.shape
    Cout = w.shape[0]
    Lout = (Lin + 2 * pad - 3) // stride + 1
    out = np.empty((B, Cout, Lout), np.float32)
    lib().orc_conv1d_k3(_p(x), _p(w), _p(b), _p(out), C.c_uint64(B), C.c_uint64(Cin), C.c_uint64(Lin), C.c_uint64(Cout),
                        C.c_uint64(stride), C.c_uint64(pad))
    return out
