"""An eager tensor with ratchet's ``Tensor`` method names, computed by the CPU oracle.

TEST INFRASTRUCTURE: lets the tests run the very same ``schedule()`` code (ratchet_b200.nn /
ratchet_b200.callers) on the CPU restatement of the reference and on the CUDA device, and compare.
Quantised matmul = dequantise then float matmul, which is what the reference's CPU device would do
(cpu/gemm.rs rejects quantised dtypes; quant.rs:132-164 provides the dequantiser).
"""
import numpy as np

from oracle import oracle as orc

F32, F16, BF16, I32, U32, Q8_0F, Q8_0H, Q4_KF, Q4_KH = range(9)
_NP = {F32: np.float32, F16: np.float16, I32: np.int32, U32: np.uint32}
_DT = {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.int32): I32, np.dtype(np.uint32): U32}


class OTensor:
    def __init__(self, data, dt=None, shape=None):
        self.a = data          # numpy array (float / int tensors) or raw uint8 buffer (quantised)
        self._dt = dt if dt is not None else _DT[data.dtype]
        self._shape = tuple(shape) if shape is not None else tuple(data.shape)

    # ---- constructors
    @staticmethod
    def from_data(data, shape=None, device=None, dt=None):
        a = np.ascontiguousarray(data)
        if shape is not None:
            a = a.reshape(shape)
        if a.ndim == 0:
            a = a.reshape(1)
        return OTensor(a.copy())

    @staticmethod
    def from_quantized(raw, dt, shape, device=None):
        return OTensor(np.ascontiguousarray(raw).view(np.uint8).reshape(-1).copy(), dt, shape)

    @staticmethod
    def zeros(shape, dt, device=None):
        return OTensor(np.zeros(shape, _NP[dt]))

    # ---- introspection
    def shape(self): return self._shape
    def rank(self): return len(self._shape)
    def dt(self): return self._dt
    def clone(self): return self
    def consume(self): pass
    def resolve(self): return self
    def to_numpy(self): return self.a

    def _dense(self):
        if self._dt in (Q8_0F, Q8_0H):
            return orc.dequantize_q8(self.a, self._shape, self._dt == Q8_0H)
        if self._dt in (Q4_KF, Q4_KH):
            return orc.dequantize_q4k(self.a, self._shape, self._dt == Q4_KH)
        return self.a

    # ---- elementwise
    def _binary(self, op, other):
        shape = np.broadcast_shapes(self._shape, other._shape)
        x = np.ascontiguousarray(np.broadcast_to(self.a, shape))
        y = np.ascontiguousarray(np.broadcast_to(other.a, shape))
        return OTensor(orc.binary(op, x, y))

    def add(self, o): return self._binary("add", o)
    def sub(self, o): return self._binary("sub", o)
    def mul(self, o): return self._binary("mul", o)
    def div(self, o): return self._binary("div", o)

    def cast(self, dt):
        if dt == self._dt:
            return self
        return OTensor(orc.cast(self.a, self._dt, dt))

    def full(self): return self.cast(F32)
    def half(self): return self.cast(F16)

    def layer_norm(self, w, b, eps): return OTensor(orc.layer_norm(self.a, w.a, None if b is None else b.a, eps))
    def rms_norm(self, w, eps): return OTensor(orc.rms_norm(self.a, w.a, eps))
    def conv1d(self, w, b, stride, padding): return OTensor(orc.conv1d_k3(self.a, w.a, None if b is None else b.a, stride, padding))
    def softmax(self, dim): return OTensor(orc.softmax(self.a, dim))
    def rope(self, dim, base, offset): return OTensor(orc.rope(self.a, dim, base, offset))

    # ---- matmul
    def matmul(self, rhs, trans_lhs=False, trans_rhs=False):
        return OTensor(orc.matmul(self._dense(), rhs.a, None, trans_lhs, trans_rhs, False))

    def gemm(self, rhs, bias, trans_lhs, trans_rhs, trans_out):
        return OTensor(orc.matmul(self._dense(), rhs.a, None if bias is None else bias.a, trans_lhs, trans_rhs, trans_out))

    # ---- data movement
    def slice(self, ranges): return OTensor(orc.slice_(self.a, [(r.start or 0, r.stop) if isinstance(r, slice) else tuple(r) for r in ranges]))
    def view(self, shape): return OTensor(self.a.reshape(shape))
    def permute(self, dims): return OTensor(orc.permute(self.a, list(dims)))
    def broadcast_to(self, shape): return OTensor(orc.broadcast(self.a, list(shape)))
    def cache(self, src, dim, offset): return OTensor(orc.cache(self.a, src.a, dim, offset))
    def index_write(self, src, start): return OTensor(orc.index_write(self.a.copy(), src.a, list(start)))

    @staticmethod
    def cat(tensors, dim): return OTensor(orc.concat([t.a for t in tensors], dim))

    def index_select(self, ids, dim):
        if self._dt in (Q8_0F, Q8_0H):
            return OTensor(orc.index_select_q8(self.a, self._shape, self._dt == Q8_0H, ids.a, dim))
        return OTensor(orc.index_select(self.a, ids.a, dim))


for _name in ("gelu", "tanh", "exp", "log", "sin", "cos", "abs", "sqrt", "relu", "floor", "ceil", "neg", "sigmoid", "silu"):
    setattr(OTensor, _name, (lambda n: lambda self: OTensor(orc.unary(n, self.a)))(_name))
