"""Thin graph builders over ``Tensor``, restating ratchet-nn (crates/ratchet-nn/src) so the model
graphs of the reference can be scheduled on the CUDA device exactly as written there.

Modules are duck-typed over the tensor class: anything with ratchet's ``Tensor`` method names works
(the tests run the same modules over a CPU-oracle tensor to get the reference result).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from . import capi


class Linear:
    """ratchet-nn/src/linear.rs:10-24: ``w.gemm(x, bias.cast(x.dt), false, true, true)`` = x W^T + b."""

    def __init__(self, w, b=None):
        self.w = w
        self.b = b

    def schedule(self, x):
        b = self.b.cast(x.dt()) if self.b is not None else None
        return self.w.gemm(x, b, False, True, True)


class Embedding:
    """ratchet-nn/src/embedding.rs:15-25: view to 1-D ids, index_select rows, view back."""

    def __init__(self, weight):
        self.weight = weight

    def schedule(self, ids):
        out_shape = list(ids.shape()) + [self.weight.shape()[-1]]
        n = 1
        for s in ids.shape():
            n *= s
        flat = ids.view([n])
        return self.weight.index_select(flat, 0).view(out_shape)


class LayerNorm:
    """ratchet-nn/src/norm.rs:37-43: upcast to f32, normalise, cast back."""

    def __init__(self, weight, bias, eps: float):
        self.weight, self.bias, self.eps = weight, bias, eps

    def schedule(self, x):
        return x.full().layer_norm(self.weight, self.bias, self.eps).cast(x.dt())


class RMSNorm:
    """ratchet-nn/src/norm.rs:63-69."""

    def __init__(self, weight, eps: float):
        self.weight, self.eps = weight, eps

    def schedule(self, x):
        return x.full().rms_norm(self.weight, self.eps).cast(x.dt())


class RotaryEmbedding:
    """ratchet-nn/src/rope.rs:24-45 (half-split pairs; ``traditional`` and ``scale`` are carried but,
    as in the reference, unused by the op)."""

    def __init__(self, dim: int, traditional: bool, base: float, scale: float):
        self.dim, self.traditional, self.base, self.scale = dim, traditional, base, scale

    def schedule(self, x, offset: int):
        return x.rope(self.dim, self.base, offset)


@dataclass
class KVEntry:
    """ratchet-nn/src/kv_cache.rs:4-19."""
    k_cache: object
    v_cache: object
    entries: int = 0


@dataclass
class KVCache:
    """ratchet-nn/src/kv_cache.rs:21-54."""
    layers: List[KVEntry] = field(default_factory=list)

    def __getitem__(self, i: int) -> KVEntry:
        return self.layers[i]

    def update(self, offset: int) -> None:
        for e in self.layers:
            e.entries += offset

    def entries(self, layer: int) -> int:
        return self.layers[layer].entries

    def reset(self) -> None:
        for e in self.layers:
            e.entries = 0
