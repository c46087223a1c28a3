"""Lazy ``Tensor`` over the CUDA device: same method names, argument meaning and error behaviour as
ratchet-core's ``Tensor`` (crates/ratchet-core/src/tensor.rs:294-510).

A ``Tensor`` owns one reference to a node of the C++ lazy graph (``rcu_lazy``).  As in the
reference, builder methods only record operations; ``resolve()`` runs them.  The reference's
methods take ``self`` by value: calling ``x.add(y)`` consumes ``x`` unless the caller wrote
``x.clone()``.  Python has no moves, so builders here borrow their operands; to let an op run in
place (the reference allows it only when the op is the operand's sole owner) drop your handle with
``Tensor.consume()`` or simply let it go out of scope before ``resolve()``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import capi
from .capi import RatchetCudaError
from .device import Device


def _u64(seq):
    return (C.c_uint64 * len(seq))(*[int(s) for s in seq])


class Tensor:
    __slots__ = ("dev", "_h")

    def __init__(self, dev: Device, handle):
        self.dev = dev
        self._h = handle

    # ------------------------------------------------------------------ lifetime
    def __del__(self):
        try:
            self.consume()
        except Exception:
            pass

    def consume(self) -> None:
        """Drop this handle's reference (what passing ``self`` by value does in the reference)."""
        if self._h is not None and self.dev.handle:
            self.dev._lib.rcu_lazy_release(self._h)
        self._h = None

    def clone(self) -> "Tensor":
        """Arc clone: a second handle to the same node (tensor.rs `#[derive(Clone)]`)."""
        self.dev._lib.rcu_lazy_retain(self._h)
        return Tensor(self.dev, self._h)

    def strong_count(self) -> int:
        return self.dev._lib.rcu_lazy_strong_count(self._h)

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def from_data(data, shape=None, device: Device = None, dt: Optional[int] = None) -> "Tensor":
        """Tensor::from_data (tensor.rs:578-616)."""
        a = np.ascontiguousarray(data)
        if shape is not None:
            a = a.reshape(shape)
        if dt is None:
            dt = capi.dt_of_numpy(a)
        shp = a.shape if a.ndim else (1,)
        h = C.c_void_p()
        device.check(device._lib.rcu_lazy_from_host(device.handle, dt, len(shp), _u64(shp), a.ctypes.data_as(C.c_void_p),
                                                    a.nbytes, C.byref(h)))
        return Tensor(device, h)

    @staticmethod
    def from_quantized(raw, dt: int, shape, device: Device) -> "Tensor":
        """Tensor::from_quantized (tensor.rs:618-628): raw bytes of a ratchet segment buffer."""
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        n = int(np.prod(shape))
        if raw.nbytes < capi.dtype_nbytes(dt, n):
            raise RatchetCudaError(capi.ERR_INVALID_ARG, "quantised buffer is smaller than its layout")
        h = C.c_void_p()
        device.check(device._lib.rcu_lazy_from_host(device.handle, dt, len(shape), _u64(shape), raw.ctypes.data_as(C.c_void_p),
                                                    raw.nbytes, C.byref(h)))
        return Tensor(device, h)

    @staticmethod
    def zeros(shape, dt: int, device: Device) -> "Tensor":
        h = C.c_void_p()
        device.check(device._lib.rcu_lazy_zeros(device.handle, dt, len(shape), _u64(shape), C.byref(h)))
        return Tensor(device, h)

    @staticmethod
    def randn(shape, device: Device, dt: int = capi.F32, seed: int = 0) -> "Tensor":
        g = np.random.Generator(np.random.PCG64(seed))
        return Tensor.from_data(g.standard_normal(shape).astype(capi.np_dtype(dt)), device=device)

    # ------------------------------------------------------------------ introspection
    def _info(self):
        t = capi.rcu_tensor()
        resolved = self.dev._lib.rcu_lazy_info(self._h, C.byref(t))
        return t, bool(resolved)

    def shape(self):
        t, _ = self._info()
        return tuple(t.shape[i] for i in range(t.rank))

    def rank(self) -> int:
        return self._info()[0].rank

    def dt(self) -> int:
        return self._info()[0].dt

    def resolved(self) -> bool:
        return self._info()[1]

    def data_ptr(self) -> int:
        return self._info()[0].data or 0

    # ------------------------------------------------------------------ builders
    def _new(self, fn, *args) -> "Tensor":
        h = C.c_void_p()
        self.dev.check(fn(*args, C.byref(h)))
        return Tensor(self.dev, h)

    def _binary(self, op: str, other: "Tensor") -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_binary, capi.BINARY_OPS[op], self._h, other._h)

    def add(self, other): return self._binary("add", other)
    def sub(self, other): return self._binary("sub", other)
    def mul(self, other): return self._binary("mul", other)
    def div(self, other): return self._binary("div", other)

    def _unary(self, op: str) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_unary, capi.UNARY_OPS[op], self._h)

    def gelu(self): return self._unary("gelu")
    def tanh(self): return self._unary("tanh")
    def exp(self): return self._unary("exp")
    def log(self): return self._unary("log")
    def sin(self): return self._unary("sin")
    def cos(self): return self._unary("cos")
    def abs(self): return self._unary("abs")
    def sqrt(self): return self._unary("sqrt")
    def relu(self): return self._unary("relu")
    def floor(self): return self._unary("floor")
    def ceil(self): return self._unary("ceil")
    def neg(self): return self._unary("neg")
    def sigmoid(self): return self._unary("sigmoid")
    def silu(self): return self._unary("silu")

    def cast(self, dst_dt: int) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_cast, self._h, dst_dt)

    def full(self) -> "Tensor":
        return self.cast(capi.F32)

    def half(self) -> "Tensor":
        return self.cast(capi.F16)

    def layer_norm(self, weight: "Tensor", bias: Optional["Tensor"], eps: float) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_norm, capi.LAYER_NORM, self._h, weight._h, bias._h if bias else None, eps, 0)

    def rms_norm(self, weight: "Tensor", eps: float) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_norm, capi.RMS_NORM, self._h, weight._h, None, eps, 0)

    def group_norm(self, num_groups: int, weight: "Tensor", bias: Optional["Tensor"], eps: float) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_norm, capi.GROUP_NORM, self._h, weight._h, bias._h if bias else None, eps, num_groups)

    def conv1d(self, weight: "Tensor", bias: Optional["Tensor"], stride: int, padding: int) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_conv1d, self._h, weight._h, bias._h if bias else None, stride, padding)

    def softmax(self, dim: int) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_softmax, self._h, dim)

    def rope(self, dim: int, base: float, offset: int) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_rope, self._h, dim, base, offset)

    def matmul(self, rhs: "Tensor", trans_lhs: bool = False, trans_rhs: bool = False) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_matmul, self._h, rhs._h, None, int(trans_lhs), int(trans_rhs), 0)

    def gemm(self, rhs: "Tensor", bias: Optional["Tensor"], trans_lhs: bool, trans_rhs: bool, trans_out: bool) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_matmul, self._h, rhs._h, bias._h if bias else None, int(trans_lhs),
                         int(trans_rhs), int(trans_out))

    def slice(self, ranges: Sequence) -> "Tensor":
        """ranges: one (start, stop) pair or Python ``slice`` per dimension (tensor.rs:421-448)."""
        shp = self.shape()
        start, stop = [], []
        for i, r in enumerate(ranges):
            if isinstance(r, slice):
                a, b = (0 if r.start is None else r.start), (shp[i] if r.stop is None else r.stop)
            else:
                a, b = r
            start.append(a)
            stop.append(b)
        if len(start) != len(shp):
            raise RatchetCudaError(capi.ERR_INVALID_ARG, "slice: one range per dimension is required")
        return self._new(self.dev._lib.rcu_lazy_slice, self._h, _u64(start), _u64(stop))

    def view(self, shape) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_view, self._h, len(shape), _u64(shape))

    @staticmethod
    def cat(tensors: Sequence["Tensor"], dim: int) -> "Tensor":
        dev = tensors[0].dev
        arr = (C.c_void_p * len(tensors))(*[t._h for t in tensors])
        h = C.c_void_p()
        dev.check(dev._lib.rcu_lazy_concat(arr, len(tensors), dim, C.byref(h)))
        return Tensor(dev, h)

    def permute(self, dims: Sequence[int]) -> "Tensor":
        if len(dims) != self.rank():
            raise RatchetCudaError(capi.ERR_INVALID_ARG, "permute: one entry per dimension is required")
        return self._new(self.dev._lib.rcu_lazy_permute, self._h, (C.c_uint32 * len(dims))(*dims))

    def cache(self, source: "Tensor", dim: int, offset: int) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_cache, self._h, source._h, dim, offset)

    def broadcast_to(self, shape) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_broadcast, self._h, len(shape), _u64(shape))

    def index_select(self, indices: "Tensor", dim: int) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_index_select, self._h, indices._h, dim)

    def index_write(self, src: "Tensor", write_start: Sequence[int]) -> "Tensor":
        return self._new(self.dev._lib.rcu_lazy_index_write, self._h, src._h, _u64(write_start))

    # ------------------------------------------------------------------ execution
    def resolve(self) -> "Tensor":
        """Tensor::resolve (tensor.rs:861-863). Asynchronous; ``to_numpy`` / ``Device.sync`` wait."""
        self.dev.check(self.dev._lib.rcu_lazy_resolve(self._h))
        return self

    def to_numpy(self) -> np.ndarray:
        """``.to(&Device::CPU)`` + ``to_vec`` (tensor.rs:949-975)."""
        t, _ = self._info()
        shape = tuple(t.shape[i] for i in range(t.rank))
        if t.dt in (capi.Q8_0F, capi.Q8_0H, capi.Q4_KF, capi.Q4_KH):
            out = np.empty(capi.dtype_nbytes(t.dt, int(np.prod(shape))), np.uint8)
        else:
            out = np.empty(shape, capi.np_dtype(t.dt))
        self.dev.check(self.dev._lib.rcu_lazy_to_host(self._h, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out


def last_resolve_stats(dev: Device) -> dict:
    s = capi.rcu_resolve_stats()
    dev._lib.rcu_last_resolve_stats(dev.handle, C.byref(s))
    return {f: getattr(s, f) for f, _ in capi.rcu_resolve_stats._fields_}
