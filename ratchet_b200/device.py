"""`Device::CUDA` and `Storage::CUDA` as seen from Python: a device handle, pooled device buffers and
the eager, op-by-op surface of the C ABI.

Mirrors ratchet-core's ``Device`` (device.rs:25-93), ``GPUBuffer`` (storage/gpu_buffer.rs) and the
per-op entry points of the resolve path.  Everything here calls ``libratchet_cuda.so``; nothing is
computed on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import capi
from .capi import RatchetCudaError


class Buffer:
    """A resolved tensor on the device: dtype, logical shape and one pooled allocation."""

    __slots__ = ("dev", "dt", "shape", "ptr", "nbytes", "_owned", "_base")

    def __init__(self, dev: "Device", dt: int, shape, ptr: int, nbytes: int, owned: bool, base=None):
        self.dev = dev
        self.dt = dt
        self.shape = tuple(int(s) for s in shape)
        self.ptr = ptr
        self.nbytes = nbytes
        self._owned = owned
        self._base = base  # keeps the owning buffer alive for views

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def desc(self) -> capi.rcu_tensor:
        return capi.describe(self.dt, self.shape, self.ptr)

    def view(self, shape) -> "Buffer":
        """Same storage, new shape (Tensor::view, tensor.rs:454-461)."""
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        if n != self.numel:
            raise RatchetCudaError(capi.ERR_INVALID_ARG, f"view: {self.shape} -> {shape} changes the element count")
        return Buffer(self.dev, self.dt, shape, self.ptr, self.nbytes, False, base=self._base or self)

    def to_numpy(self) -> np.ndarray:
        """Tensor::to(Device::CPU): blocking device-to-host copy."""
        if self.dt in (capi.Q8_0F, capi.Q8_0H, capi.Q4_KF, capi.Q4_KH):
            out = np.empty(self.nbytes, np.uint8)
        else:
            out = np.empty(self.shape, capi.np_dtype(self.dt))
        self.dev.d2h(out, self.ptr, out.nbytes)
        return out

    def free(self) -> None:
        if self._owned and self.ptr:
            self.dev._free(self.ptr)
            self.ptr = 0
            self._owned = False

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Device:
    """One CUDA device + stream + caching allocator (``rcu_device``)."""

    def __init__(self, ordinal: int = 0, stream: Optional[int] = None):
        self._lib = capi.lib()
        handle = C.c_void_p()
        if stream is None:
            st = self._lib.rcu_device_create(ordinal, C.byref(handle))
        else:
            st = self._lib.rcu_device_create_on_stream(ordinal, C.c_void_p(stream), C.byref(handle))
        if st != capi.OK:
            raise RatchetCudaError(st, f"cannot open CUDA device {ordinal} (this library needs an sm_100 GPU; "
                                       "there is no CPU fallback)")
        self.handle = handle
        self.ordinal = ordinal

    # ------------------------------------------------------------------ plumbing
    def close(self) -> None:
        if self.handle:
            self._lib.rcu_device_destroy(self.handle)
            self.handle = None

    def check(self, st: int) -> None:
        if st != capi.OK:
            msg = self._lib.rcu_last_error(self.handle)
            raise RatchetCudaError(st, msg.decode() if msg else "")

    def sync(self) -> None:
        self.check(self._lib.rcu_sync(self.handle))

    @property
    def launches(self) -> int:
        return self._lib.rcu_launch_count(self.handle)

    @property
    def sm_count(self) -> int:
        return self._lib.rcu_sm_count(self.handle)

    def pool_stats(self):
        a, b = C.c_uint64(), C.c_uint64()
        self._lib.rcu_pool_stats(self.handle, C.byref(a), C.byref(b))
        return a.value, b.value

    def _alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self._lib.rcu_alloc(self.handle, nbytes, C.byref(p)))
        return p.value

    def _free(self, ptr: int) -> None:
        if self.handle:
            self._lib.rcu_free(self.handle, C.c_void_p(ptr))

    def h2d(self, ptr: int, host: np.ndarray, nbytes: Optional[int] = None) -> None:
        self.check(self._lib.rcu_h2d(self.handle, C.c_void_p(ptr), host.ctypes.data_as(C.c_void_p),
                                     host.nbytes if nbytes is None else nbytes))

    def d2h(self, host: np.ndarray, ptr: int, nbytes: int) -> None:
        self.check(self._lib.rcu_d2h(self.handle, host.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), nbytes))

    def d2h_async(self, host: np.ndarray, ptr: int, nbytes: int) -> None:
        """Device-to-host copy that does not wait (pinned `host`; valid after the next sync on this handle)."""
        self.check(self._lib.rcu_d2h_async(self.handle, host.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), nbytes))

    def wait_for(self, other: "Device") -> None:
        """Work queued on this handle from now on starts after what is queued on `other` (same GPU) so far."""
        self.check(self._lib.rcu_stream_wait(self.handle, other.handle))

    # ------------------------------------------------------------------ storage
    def empty(self, dt: int, shape) -> Buffer:
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        nbytes = capi.dtype_nbytes(dt, n)
        return Buffer(self, dt, shape, self._alloc(nbytes), nbytes, True)

    def zeros(self, dt: int, shape) -> Buffer:
        b = self.empty(dt, shape)
        self.check(self._lib.rcu_memset(self.handle, C.c_void_p(b.ptr), 0, b.nbytes))
        return b

    def from_numpy(self, a: np.ndarray, dt: Optional[int] = None) -> Buffer:
        """Tensor::from_data (tensor.rs:578-616): host array -> device buffer."""
        a = np.ascontiguousarray(a)
        if dt is None:
            dt = capi.dt_of_numpy(a)
        shape = a.shape if a.ndim else (1,)
        b = self.empty(dt, shape)
        self.h2d(b.ptr, a, a.nbytes)
        return b

    def from_quantized(self, raw: np.ndarray, dt: int, shape) -> Buffer:
        """Tensor::from_quantized (tensor.rs:618-628): a ratchet segment buffer as raw bytes."""
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        b = self.empty(dt, shape)
        if raw.nbytes < b.nbytes:
            raise RatchetCudaError(capi.ERR_INVALID_ARG, f"quantised buffer has {raw.nbytes} bytes, layout needs {b.nbytes}")
        self.h2d(b.ptr, raw, b.nbytes)
        return b

    def wrap(self, dt: int, shape, ptr: int) -> Buffer:
        """Describe device memory owned by someone else (e.g. a framework tensor's data pointer)."""
        n = 1
        for s in shape:
            n *= int(s)
        return Buffer(self, dt, shape, ptr, capi.dtype_nbytes(dt, n), False)

    # ------------------------------------------------------------------ ops (eager, one C-ABI call each)
    def _ref(self, b: Optional[Buffer]):
        return None if b is None else C.byref(b.desc())

    def dequantize(self, src: Buffer, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(capi.activation_dtype(src.dt), src.shape)
        self.check(self._lib.rcu_dequantize(self.handle, self._ref(src), self._ref(out)))
        return out

    def set_debug(self, no_reuse: bool = False, profile: bool = False, log: bool = False) -> None:
        """Debug switches of the lazy resolver: one buffer per tensor and nothing in place (the reference's
        RATCHET_DEBUG), and a per-op timing table (its `gpu-profiling` feature)."""
        self.check(self._lib.rcu_set_debug(self.handle, (capi.DEBUG_NO_REUSE if no_reuse else 0) | (capi.DEBUG_PROFILE if profile else 0) |
                                            (capi.DEBUG_LOG if log else 0)))

    def profile_report(self, reset: bool = True) -> str:
        """The per-op table collected while the profile switch was on: kernel, count, total us, %, GB/s."""
        n = self._lib.rcu_profile_report(self.handle, None, 0, 0)
        buf = C.create_string_buffer(int(n))
        self._lib.rcu_profile_report(self.handle, buf, n, int(reset))
        return buf.value.decode()

    def set_constant_weights(self, on: bool = True) -> None:
        """Promise that nothing in flight writes the weight operands of the GEMVs that follow (a loaded model's
        Linear weights): they are then launched as programmatic dependents and start fetching weights early."""
        self.check(self._lib.rcu_set_constant_weights(self.handle, int(bool(on))))

    def set_wait_limit_ns(self, ns: int) -> None:
        """How long a device-side wait may last before it gives up (default two seconds)."""
        self.check(self._lib.rcu_set_wait_limit_ns(self.handle, int(ns)))

    def quantize(self, src: Buffer, out: Optional[Buffer] = None) -> Buffer:
        """quant.rs:51-99 on the device: f32 -> Q8_0F, f16 -> Q8_0H, same shape."""
        out = out or self.empty(capi.Q8_0H if src.dt == capi.F16 else capi.Q8_0F, src.shape)
        self.check(self._lib.rcu_quantize_device(self.handle, self._ref(src), self._ref(out)))
        return out

    def matmul_shape(self, lhs: Buffer, rhs: Buffer, trans_lhs=False, trans_rhs=False, trans_dst=False):
        d = capi.rcu_tensor()
        st = self._lib.rcu_matmul_dst_shape(self._ref(lhs), self._ref(rhs), int(trans_lhs), int(trans_rhs), int(trans_dst),
                                            C.byref(d))
        if st != capi.OK:
            raise RatchetCudaError(st, f"matmul: incompatible shapes {lhs.shape} x {rhs.shape}")
        return tuple(d.shape[i] for i in range(d.rank)), d.dt

    def matmul(self, lhs: Buffer, rhs: Buffer, bias: Optional[Buffer] = None, trans_lhs=False, trans_rhs=False,
               trans_dst=False, out: Optional[Buffer] = None) -> Buffer:
        if out is None:
            shape, dt = self.matmul_shape(lhs, rhs, trans_lhs, trans_rhs, trans_dst)
            out = self.empty(dt, shape)
        self.check(self._lib.rcu_matmul(self.handle, self._ref(lhs), self._ref(rhs), self._ref(bias), int(trans_lhs),
                                        int(trans_rhs), int(trans_dst), self._ref(out)))
        return out

    def binary(self, op: str, a: Buffer, b: Buffer, out: Optional[Buffer] = None) -> Buffer:
        if out is None:
            shape = np.broadcast_shapes(a.shape, b.shape)
            out = self.empty(a.dt, shape)
        self.check(self._lib.rcu_binary(self.handle, capi.BINARY_OPS[op], self._ref(a), self._ref(b), self._ref(out)))
        return out

    def unary(self, op: str, x: Buffer, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, x.shape)
        self.check(self._lib.rcu_unary(self.handle, capi.UNARY_OPS[op], self._ref(x), self._ref(out)))
        return out

    def cast(self, x: Buffer, dt: int, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(dt, x.shape)
        self.check(self._lib.rcu_cast(self.handle, self._ref(x), self._ref(out)))
        return out

    def norm(self, kind: int, x: Buffer, scale: Buffer, bias: Optional[Buffer], eps: float, groups: int = 0,
             out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, x.shape)
        self.check(self._lib.rcu_norm(self.handle, kind, self._ref(x), self._ref(scale), self._ref(bias), eps, groups,
                                      self._ref(out)))
        return out

    def softmax(self, x: Buffer, dim: int, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, x.shape)
        self.check(self._lib.rcu_softmax(self.handle, self._ref(x), dim, self._ref(out)))
        return out

    def reduce(self, kind: int, x: Buffer, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, x.shape[:-1] if len(x.shape) > 1 else (1,))
        self.check(self._lib.rcu_reduce(self.handle, kind, self._ref(x), self._ref(out)))
        return out

    def rope(self, x: Buffer, dim: int, base: float, offset: int, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, x.shape)
        self.check(self._lib.rcu_rope(self.handle, self._ref(x), dim, base, offset, self._ref(out)))
        return out

    def concat(self, inputs: Sequence[Buffer], dim: int, out: Optional[Buffer] = None) -> Buffer:
        if out is None:
            shape = list(inputs[0].shape)
            shape[dim] = sum(t.shape[dim] for t in inputs)
            out = self.empty(inputs[0].dt, shape)
        descs = [t.desc() for t in inputs]
        arr = (capi._T * len(descs))(*[C.pointer(d) for d in descs])
        self.check(self._lib.rcu_concat(self.handle, arr, len(descs), dim, self._ref(out)))
        return out

    def index_select(self, src: Buffer, ids: Buffer, dim: int, out: Optional[Buffer] = None) -> Buffer:
        if out is None:
            shape = list(src.shape)
            shape[dim] = ids.shape[0]
            out = self.empty(capi.activation_dtype(src.dt), shape)
        self.check(self._lib.rcu_index_select(self.handle, self._ref(src), self._ref(ids), dim, self._ref(out)))
        return out

    def permute(self, x: Buffer, perm: Sequence[int], out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, [x.shape[p] for p in perm])
        self.check(self._lib.rcu_permute(self.handle, self._ref(x), (C.c_uint32 * len(perm))(*perm), self._ref(out)))
        return out

    def slice(self, x: Buffer, ranges, out: Optional[Buffer] = None) -> Buffer:
        start = [r[0] for r in ranges]
        stop = [r[1] for r in ranges]
        out = out or self.empty(x.dt, [b - a for a, b in ranges])
        n = len(ranges)
        self.check(self._lib.rcu_slice(self.handle, self._ref(x), (C.c_uint64 * n)(*start), (C.c_uint64 * n)(*stop),
                                       self._ref(out)))
        return out

    def broadcast(self, x: Buffer, shape, out: Optional[Buffer] = None) -> Buffer:
        out = out or self.empty(x.dt, shape)
        self.check(self._lib.rcu_broadcast(self.handle, self._ref(x), self._ref(out)))
        return out

    def cache(self, cache: Buffer, src: Buffer, dim: int, offset: int, out: Optional[Buffer] = None, materialise=True):
        if out is None and materialise:
            shape = list(cache.shape)
            shape[dim] = offset + src.shape[dim]
            out = self.empty(cache.dt, shape)
        self.check(self._lib.rcu_cache(self.handle, self._ref(cache), self._ref(src), dim, offset, self._ref(out)))
        return out

    def index_write(self, dst: Buffer, src: Buffer, start: Sequence[int]) -> Buffer:
        self.check(self._lib.rcu_index_write(self.handle, self._ref(dst), self._ref(src), (C.c_uint64 * len(start))(*start)))
        return dst

    def conv1d(self, x: Buffer, w: Buffer, bias: Optional[Buffer], stride: int, padding: int, out: Optional[Buffer] = None):
        if out is None:
            lout = (x.shape[2] + 2 * padding - 3) // stride + 1
            out = self.empty(x.dt, (x.shape[0], w.shape[0], lout))
        self.check(self._lib.rcu_conv1d(self.handle, self._ref(x), self._ref(w), self._ref(bias), stride, padding,
                                        self._ref(out)))
        return out
