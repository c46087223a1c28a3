"""ctypes binding of ``libratchet_cuda.so`` — one Python function per C-ABI symbol of
``include/ratchet_cuda.h`` plus the small amount of glue needed to describe tensors.

There is no fallback: importing works without a GPU (so symbol tables can be checked), but every
compute call needs the library and a B200, and raises :class:`RatchetCudaError` otherwise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libratchet_cuda.so")

RCU_MAX_RANK = 4

# rcu_status
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_BOUNDS, ERR_INPLACE = range(9)
_STATUS_NAMES = ["RCU_OK", "RCU_ERR_INVALID_ARG", "RCU_ERR_UNSUPPORTED", "RCU_ERR_OOM", "RCU_ERR_CUDA", "RCU_ERR_NCCL",
                 "RCU_ERR_TIMEOUT", "RCU_ERR_BOUNDS", "RCU_ERR_INPLACE"]

# rcu_dtype (ratchet-core/src/dtype/mod.rs:11-23)
F32, F16, BF16, I32, U32, Q8_0F, Q8_0H, Q4_KF, Q4_KH = range(9)
DTYPE_NAMES = ["F32", "F16", "BF16", "I32", "U32", "Q8_0F", "Q8_0H", "Q4_KF", "Q4_KH"]
_NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16, I32: np.int32, U32: np.uint32}
_DT_OF_NP = {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.int32): I32, np.dtype(np.uint32): U32}

BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3}
UNARY_OPS = {"gelu": 0, "tanh": 1, "exp": 2, "log": 3, "sin": 4, "cos": 5, "abs": 6, "sqrt": 7, "relu": 8, "floor": 9,
             "ceil": 10, "neg": 11, "silu": 12, "sigmoid": 13}
LAYER_NORM, RMS_NORM, GROUP_NORM = 0, 1, 2
DEBUG_NO_REUSE, DEBUG_PROFILE, DEBUG_LOG = 1, 2, 4
REDUCE_SUM, REDUCE_MAX, REDUCE_MEAN = 0, 1, 2


class RatchetCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        name = _STATUS_NAMES[status] if 0 <= status < len(_STATUS_NAMES) else str(status)
        super().__init__(f"{name}: {message}")
        self.status = status


class rcu_tensor(C.Structure):
    _fields_ = [("dt", C.c_int32), ("rank", C.c_uint32), ("shape", C.c_uint64 * RCU_MAX_RANK), ("data", C.c_void_p)]


class rcu_resolve_stats(C.Structure):
    _fields_ = [("nodes", C.c_uint32), ("launched", C.c_uint32), ("inplace", C.c_uint32), ("buffers", C.c_uint32),
                ("planned_bytes", C.c_uint64), ("naive_bytes", C.c_uint64)]


class rcu_decoder_config(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("d_model", C.c_uint32), ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("ffn", C.c_uint32), ("vocab", C.c_uint32), ("max_cache", C.c_uint32),
                ("rope_dim", C.c_uint32), ("rope_base", C.c_float), ("rms_eps", C.c_float), ("weight_dt", C.c_int32)]


class rcu_gguf_tensor_info(C.Structure):
    _fields_ = [("name", C.c_char_p), ("rank", C.c_uint32), ("shape", C.c_uint64 * 4), ("ggml_type", C.c_uint32), ("numel", C.c_uint64),
                ("file_bytes", C.c_uint64)]


class rcu_decoder_layer(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("qkv", C.c_void_p), ("o", C.c_void_p), ("ffn_norm", C.c_void_p),
                ("gate_up", C.c_void_p), ("down", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


_T = C.POINTER(rcu_tensor)
_DEV = C.c_void_p
_LZ = C.c_void_p
_u64p = C.POINTER(C.c_uint64)
_u32p = C.POINTER(C.c_uint32)

# symbol -> (restype, argtypes); the keys are exactly the functions declared in include/ratchet_cuda.h
SIGNATURES = {
    "rcu_device_create": (C.c_int, [C.c_int, C.POINTER(_DEV)]),
    "rcu_device_create_on_stream": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(_DEV)]),
    "rcu_device_destroy": (None, [_DEV]),
    "rcu_last_error": (C.c_char_p, [_DEV]),
    "rcu_launch_count": (C.c_uint64, [_DEV]),
    "rcu_sm_count": (C.c_int, [_DEV]),
    "rcu_set_debug": (C.c_int, [_DEV, C.c_uint32]),
    "rcu_profile_report": (C.c_uint64, [_DEV, C.c_char_p, C.c_uint64, C.c_int]),
    "rcu_alloc": (C.c_int, [_DEV, C.c_uint64, C.POINTER(C.c_void_p)]),
    "rcu_free": (C.c_int, [_DEV, C.c_void_p]),
    "rcu_pool_trim": (C.c_int, [_DEV]),
    "rcu_pool_stats": (None, [_DEV, _u64p, _u64p]),
    "rcu_h2d": (C.c_int, [_DEV, C.c_void_p, C.c_void_p, C.c_uint64]),
    "rcu_d2h": (C.c_int, [_DEV, C.c_void_p, C.c_void_p, C.c_uint64]),
    "rcu_d2h_async": (C.c_int, [_DEV, C.c_void_p, C.c_void_p, C.c_uint64]),
    "rcu_stream_wait": (C.c_int, [_DEV, _DEV]),
    "rcu_d2d": (C.c_int, [_DEV, C.c_void_p, C.c_void_p, C.c_uint64]),
    "rcu_memset": (C.c_int, [_DEV, C.c_void_p, C.c_int, C.c_uint64]),
    "rcu_sync": (C.c_int, [_DEV]),
    "rcu_set_wait_limit_ns": (C.c_int, [_DEV, C.c_uint64]),
    "rcu_set_constant_weights": (C.c_int, [_DEV, C.c_int]),
    "rcu_dtype_nbytes": (C.c_uint64, [C.c_int32, C.c_uint64]),
    "rcu_dtype_segments": (C.c_int, [C.c_int32, C.c_uint64, _u64p]),
    "rcu_activation_dtype": (C.c_int32, [C.c_int32]),
    "rcu_dequantize": (C.c_int, [_DEV, _T, _T]),
    "rcu_quantize": (C.c_int, [C.c_int32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "rcu_quantize_device": (C.c_int, [_DEV, _T, _T]),
    "rcu_matmul": (C.c_int, [_DEV, _T, _T, _T, C.c_int, C.c_int, C.c_int, _T]),
    "rcu_matmul_dst_shape": (C.c_int, [_T, _T, C.c_int, C.c_int, C.c_int, _T]),
    "rcu_binary": (C.c_int, [_DEV, C.c_int, _T, _T, _T]),
    "rcu_unary": (C.c_int, [_DEV, C.c_int, _T, _T]),
    "rcu_cast": (C.c_int, [_DEV, _T, _T]),
    "rcu_norm": (C.c_int, [_DEV, C.c_int, _T, _T, _T, C.c_float, C.c_uint32, _T]),
    "rcu_softmax": (C.c_int, [_DEV, _T, C.c_uint32, _T]),
    "rcu_reduce": (C.c_int, [_DEV, C.c_int, _T, _T]),
    "rcu_rope": (C.c_int, [_DEV, _T, C.c_uint32, C.c_float, C.c_uint32, _T]),
    "rcu_concat": (C.c_int, [_DEV, C.POINTER(_T), C.c_uint32, C.c_uint32, _T]),
    "rcu_index_select": (C.c_int, [_DEV, _T, _T, C.c_uint32, _T]),
    "rcu_permute": (C.c_int, [_DEV, _T, _u32p, _T]),
    "rcu_slice": (C.c_int, [_DEV, _T, _u64p, _u64p, _T]),
    "rcu_broadcast": (C.c_int, [_DEV, _T, _T]),
    "rcu_cache": (C.c_int, [_DEV, _T, _T, C.c_uint32, C.c_uint32, _T]),
    "rcu_index_write": (C.c_int, [_DEV, _T, _T, _u64p]),
    "rcu_conv1d": (C.c_int, [_DEV, _T, _T, _T, C.c_uint32, C.c_uint32, _T]),
    # lazy tensor graph
    "rcu_lazy_from_host": (C.c_int, [_DEV, C.c_int32, C.c_uint32, _u64p, C.c_void_p, C.c_uint64, C.POINTER(_LZ)]),
    "rcu_lazy_zeros": (C.c_int, [_DEV, C.c_int32, C.c_uint32, _u64p, C.POINTER(_LZ)]),
    "rcu_lazy_wrap": (C.c_int, [_DEV, _T, C.POINTER(_LZ)]),
    "rcu_lazy_retain": (None, [_LZ]),
    "rcu_lazy_release": (None, [_LZ]),
    "rcu_lazy_info": (C.c_int, [_LZ, _T]),
    "rcu_lazy_strong_count": (C.c_uint32, [_LZ]),
    "rcu_lazy_binary": (C.c_int, [C.c_int, _LZ, _LZ, C.POINTER(_LZ)]),
    "rcu_lazy_unary": (C.c_int, [C.c_int, _LZ, C.POINTER(_LZ)]),
    "rcu_lazy_cast": (C.c_int, [_LZ, C.c_int32, C.POINTER(_LZ)]),
    "rcu_lazy_norm": (C.c_int, [C.c_int, _LZ, _LZ, _LZ, C.c_float, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_softmax": (C.c_int, [_LZ, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_rope": (C.c_int, [_LZ, C.c_uint32, C.c_float, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_matmul": (C.c_int, [_LZ, _LZ, _LZ, C.c_int, C.c_int, C.c_int, C.POINTER(_LZ)]),
    "rcu_lazy_conv1d": (C.c_int, [_LZ, _LZ, _LZ, C.c_uint32, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_view": (C.c_int, [_LZ, C.c_uint32, _u64p, C.POINTER(_LZ)]),
    "rcu_lazy_slice": (C.c_int, [_LZ, _u64p, _u64p, C.POINTER(_LZ)]),
    "rcu_lazy_permute": (C.c_int, [_LZ, _u32p, C.POINTER(_LZ)]),
    "rcu_lazy_broadcast": (C.c_int, [_LZ, C.c_uint32, _u64p, C.POINTER(_LZ)]),
    "rcu_lazy_concat": (C.c_int, [C.POINTER(_LZ), C.c_uint32, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_index_select": (C.c_int, [_LZ, _LZ, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_cache": (C.c_int, [_LZ, _LZ, C.c_uint32, C.c_uint32, C.POINTER(_LZ)]),
    "rcu_lazy_index_write": (C.c_int, [_LZ, _LZ, _u64p, C.POINTER(_LZ)]),
    "rcu_lazy_id": (C.c_uint64, [_LZ]),
    "rcu_lazy_execution_order": (C.c_int, [_LZ, _u64p, C.c_uint32, _u32p]),
    "rcu_lazy_resolve": (C.c_int, [_LZ]),
    "rcu_lazy_to_host": (C.c_int, [_LZ, C.c_void_p, C.c_uint64]),
    "rcu_last_resolve_stats": (None, [_DEV, C.POINTER(rcu_resolve_stats)]),
    # fused decode step
    # GGUF files (host side)
    "rcu_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "rcu_gguf_close": (None, [C.c_void_p]),
    "rcu_gguf_last_error": (C.c_char_p, []),
    "rcu_gguf_version": (C.c_uint32, [C.c_void_p]),
    "rcu_gguf_tensor_count": (C.c_uint64, [C.c_void_p]),
    "rcu_gguf_find": (C.c_int64, [C.c_void_p, C.c_char_p]),
    "rcu_gguf_tensor": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(rcu_gguf_tensor_info)]),
    "rcu_gguf_meta_u64": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "rcu_gguf_meta_f64": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_double)]),
    "rcu_gguf_meta_str": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_uint64]),
    "rcu_gguf_target_dtype": (C.c_int32, [C.c_uint32, C.c_int]),
    "rcu_gguf_transcode": (C.c_int, [C.c_void_p, C.c_uint64, C.c_int32, C.c_void_p, C.c_uint64]),
    "rcu_decoder_create": (C.c_int, [_DEV, C.POINTER(rcu_decoder_config), C.POINTER(rcu_decoder_layer), C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.POINTER(C.c_void_p)]),
    "rcu_decoder_create_sharded": (C.c_int, [_DEV, C.c_void_p, C.POINTER(rcu_decoder_config), C.POINTER(rcu_decoder_layer), C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "rcu_decoder_destroy": (None, [C.c_void_p]),
    "rcu_decoder_set_position": (C.c_int, [C.c_void_p, C.c_uint32]),
    "rcu_decoder_position": (C.c_uint32, [C.c_void_p]),
    "rcu_decoder_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rcu_decoder_kernels_per_step": (C.c_uint32, [C.c_void_p]),
    "rcu_decoder_profile_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _u64p, C.c_uint32, _u32p]),
    "rcu_attn_decode_static": (C.c_int, [_DEV, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                         C.c_uint32, C.c_float, C.c_uint32, C.c_void_p]),
    "rcu_comm_create": (C.c_int, [_DEV, C.c_int, C.c_int, C.c_uint64, C.POINTER(C.c_void_p)]),
    "rcu_comm_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rcu_comm_import": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "rcu_comm_import_local": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "rcu_comm_destroy": (None, [C.c_void_p]),
    "rcu_comm_rank": (C.c_int, [C.c_void_p]),
    "rcu_comm_world": (C.c_int, [C.c_void_p]),
    "rcu_gemv_q8_allgather": (C.c_int, [C.c_void_p, _T, _T, _T, C.POINTER(C.c_void_p)]),
    "rcu_attn_decode": (C.c_int, [_DEV, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                  C.c_uint32, C.c_float, C.c_uint32, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library (built in-tree by ``ratchet_b200._build``). Fails loudly if absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RatchetCudaError(ERR_CUDA, f"{LIB_PATH} is missing: run `python -m ratchet_b200._build` "
                                             "(there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def dtype_nbytes(dt: int, numel: int) -> int:
    return lib().rcu_dtype_nbytes(dt, numel)


def dtype_segments(dt: int, numel: int):
    off = (C.c_uint64 * 4)()
    n = lib().rcu_dtype_segments(dt, numel, off)
    return [off[i] for i in range(n)]


def quantize(x: np.ndarray) -> np.ndarray:
    """``quantize`` of ratchet-core/src/quant.rs:51-99 on the host: f32 input -> Q8_0F buffer, f16 input ->
    Q8_0H buffer (a uint8 array in ratchet's segment layout)."""
    x = np.ascontiguousarray(x)
    if x.dtype not in (np.float32, np.float16):
        raise RatchetCudaError(ERR_INVALID_ARG, f"quantize: {x.dtype} input (f32 or f16 expected)")
    dt = Q8_0H if x.dtype == np.float16 else Q8_0F
    out = np.empty(dtype_nbytes(dt, x.size), np.uint8)
    st = lib().rcu_quantize(dt, x.ctypes.data_as(C.c_void_p), x.size, out.ctypes.data_as(C.c_void_p), out.size)
    if st != OK:
        raise RatchetCudaError(st, f"rcu_quantize({DTYPE_NAMES[dt]}, numel={x.size})")
    return out


def activation_dtype(dt: int) -> int:
    return lib().rcu_activation_dtype(dt)


def np_dtype(dt: int):
    return _NP_OF[dt]


def dt_of_numpy(a: np.ndarray) -> int:
    return _DT_OF_NP[a.dtype]


def describe(dt: int, shape, ptr: int) -> rcu_tensor:
    shape = tuple(int(s) for s in shape)
    if not 1 <= len(shape) <= RCU_MAX_RANK:
        raise RatchetCudaError(ERR_INVALID_ARG, f"rank {len(shape)} is outside 1..{RCU_MAX_RANK}")
    t = rcu_tensor()
    t.dt = dt
    t.rank = len(shape)
    for i, s in enumerate(shape):
        t.shape[i] = s
    t.data = ptr
    return t
