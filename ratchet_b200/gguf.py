"""GGUF files: header / tensor directory / metadata and the transcode of ggml blocks into ratchet's
segment layout (``rcu_gguf_*``; ratchet-loader/src/gguf/gguf.rs:422-509, gguf/dtype.rs:39-198).

``GGUFFile`` needs no GPU: it maps the file and transcodes into host arrays.  ``load`` uploads one
tensor to a ``Device`` as the buffer the kernels read (what ``Header::tensor`` does in the reference).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import capi
from .capi import RatchetCudaError

GGML_F32, GGML_F16, GGML_Q8_0, GGML_Q4_K = 0, 1, 8, 12


@dataclass(frozen=True)
class GGUFTensor:
    index: int
    name: str
    shape: Tuple[int, ...]        # ratchet order (outermost first)
    ggml_type: int
    numel: int
    file_bytes: int


class GGUFFile:
    def __init__(self, path: str):
        self._lib = capi.lib()
        h = C.c_void_p()
        st = self._lib.rcu_gguf_open(path.encode(), C.byref(h))
        if st != capi.OK:
            raise RatchetCudaError(st, self._lib.rcu_gguf_last_error().decode())
        self._h = h
        self.version = int(self._lib.rcu_gguf_version(h))
        self.tensors: Dict[str, GGUFTensor] = {}
        info = capi.rcu_gguf_tensor_info()
        for i in range(self._lib.rcu_gguf_tensor_count(h)):
            self._check(self._lib.rcu_gguf_tensor(h, i, C.byref(info)))
            t = GGUFTensor(i, info.name.decode(), tuple(int(info.shape[d]) for d in range(info.rank)), int(info.ggml_type),
                           int(info.numel), int(info.file_bytes))
            self.tensors[t.name] = t

    def close(self) -> None:
        if self._h is not None:
            self._lib.rcu_gguf_close(self._h)
        self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, st: int) -> None:
        if st != capi.OK:
            raise RatchetCudaError(st, self._lib.rcu_gguf_last_error().decode())

    # ------------------------------------------------------------------ metadata
    def meta_int(self, key: str) -> int:
        v = C.c_uint64()
        self._check(self._lib.rcu_gguf_meta_u64(self._h, key.encode(), C.byref(v)))
        return int(v.value)

    def meta_float(self, key: str) -> float:
        v = C.c_double()
        self._check(self._lib.rcu_gguf_meta_f64(self._h, key.encode(), C.byref(v)))
        return float(v.value)

    def meta_str(self, key: str) -> str:
        buf = C.create_string_buffer(4096)
        self._check(self._lib.rcu_gguf_meta_str(self._h, key.encode(), buf, len(buf)))
        return buf.value.decode()

    # ------------------------------------------------------------------ tensors
    def target_dtype(self, name: str, f16_device: bool = True) -> int:
        """The dtype ``ratchet_from_gguf`` loads this tensor as (f16 scales on an f16-capable device)."""
        dt = self._lib.rcu_gguf_target_dtype(self.tensors[name].ggml_type, int(f16_device))
        if dt < 0:
            raise RatchetCudaError(capi.ERR_UNSUPPORTED, f"unsupported ggml dtype {self.tensors[name].ggml_type} ({name})")
        return int(dt)

    def transcode(self, name: str, dt: Optional[int] = None) -> np.ndarray:
        """The tensor in ratchet's layout as a host array: uint8 bytes for quantised dtypes, a shaped
        float array otherwise."""
        t = self.tensors[name]
        dt = self.target_dtype(name) if dt is None else dt
        nbytes = capi.dtype_nbytes(dt, t.numel)
        out = np.zeros(nbytes, np.uint8)
        self._check(self._lib.rcu_gguf_transcode(self._h, t.index, dt, out.ctypes.data_as(C.c_void_p), nbytes))
        if dt == capi.F32:
            return out[: t.numel * 4].view(np.float32).reshape(t.shape)
        if dt == capi.F16:
            return out[: t.numel * 2].view(np.float16).reshape(t.shape)     # the buffer itself is padded to 4 bytes
        return out

    def load(self, name: str, dev, f16_device: bool = True):
        """Upload one tensor to ``dev`` (``Header::tensor``, gguf.rs:497-509)."""
        t = self.tensors[name]
        dt = self.target_dtype(name, f16_device)
        host = self.transcode(name, dt)
        if dt in (capi.F32, capi.F16):
            return dev.from_numpy(host)
        return dev.from_quantized(host, dt, t.shape)
