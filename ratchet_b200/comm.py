"""Row-sharding of a Linear over the GPUs of one node and the fused GEMV + all-gather.

The reference is single-device; this is the sharding its ``Linear`` (ratchet-nn/src/linear.rs:17-24)
admits.  ``torch.distributed`` is used only as plumbing to exchange 64-byte IPC handles once; the data
path is the CUDA library's own (``rcu_gemv_q8_allgather``: peer stores over NVLink from the GEMV's
last CTA, flag wait on the consumer).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import capi
from .capi import RatchetCudaError
from .device import Buffer, Device


def shard_rows(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [begin, end) of rank `rank`: equal contiguous slices (n_rows must divide by world)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def _align256(n: int) -> int:
    return (n + 255) // 256 * 256


def shard_q8(buf: np.ndarray, dt: int, n_rows: int, k: int, rank: int, world: int) -> np.ndarray:
    """The rank's rows of a ratchet Q8_0 buffer W[n_rows, k] as a ratchet buffer of their own
    (segments re-padded to 256 bytes, ratchet-core/src/dtype/blocks.rs:69-82).  Blocks of 32 run along
    k inside a row, so a row split never cuts a block."""
    if dt not in (capi.Q8_0F, capi.Q8_0H):
        raise ValueError("shard_q8 takes Q8_0F / Q8_0H buffers")
    if k % 32:
        raise ValueError("k must hold whole 32-element blocks")
    fp = 4 if dt == capi.Q8_0F else 2
    raw = np.ascontiguousarray(buf).view(np.uint8).reshape(-1)
    r0, r1 = shard_rows(n_rows, rank, world)
    rows = r1 - r0
    qs = raw[r0 * k: r1 * k]
    d_off = _align256(n_rows * k)
    per_row = (k // 32) * fp
    ds = raw[d_off + r0 * per_row: d_off + r1 * per_row]
    out = np.zeros(_align256(rows * k) + _align256(rows * per_row), np.uint8)
    out[: rows * k] = qs
    out[_align256(rows * k): _align256(rows * k) + rows * per_row] = ds
    return out


def take_rows_q8(buf: np.ndarray, dt: int, n_rows: int, k: int, ranges: Sequence[Tuple[int, int]]) -> np.ndarray:
    """Rows [a, b) for each (a, b) of `ranges`, in that order, of a ratchet Q8_0 buffer W[n_rows, k], as a
    ratchet buffer of their own.  shard_q8 is the single-range case."""
    if dt not in (capi.Q8_0F, capi.Q8_0H):
        raise ValueError("take_rows_q8 takes Q8_0F / Q8_0H buffers")
    if k % 32:
        raise ValueError("k must hold whole 32-element blocks")
    fp = 4 if dt == capi.Q8_0F else 2
    raw = np.ascontiguousarray(buf).view(np.uint8).reshape(-1)
    d_off = _align256(n_rows * k)
    per_row = (k // 32) * fp
    for a, b in ranges:
        if not 0 <= a <= b <= n_rows:
            raise ValueError(f"rows [{a}, {b}) outside [0, {n_rows})")
    rows = sum(b - a for a, b in ranges)
    out = np.zeros(_align256(rows * k) + _align256(rows * per_row), np.uint8)
    q_at, d_at = 0, _align256(rows * k)
    for a, b in ranges:
        n = b - a
        out[q_at: q_at + n * k] = raw[a * k: b * k]
        out[d_at: d_at + n * per_row] = raw[d_off + a * per_row: d_off + b * per_row]
        q_at += n * k
        d_at += n * per_row
    return out


def decoder_shard_ranges(n_heads: int, n_kv_heads: int, head_dim: int, d_model: int, ffn: int, vocab: int, rank: int,
                         world: int) -> dict:
    """Row ranges of each Linear that rank `rank` of `world` owns in the sharded decode step
    (rcu_decoder_create_sharded): attention is split by heads (q, k and v rows of the rank's heads),
    the gated MLP by ffn columns (gate rows then up rows of the rank's columns), every other Linear and
    the logits by contiguous output rows."""
    for name, n in (("n_heads", n_heads), ("n_kv_heads", n_kv_heads), ("d_model", d_model), ("ffn", ffn), ("vocab", vocab)):
        if n % world:
            raise ValueError(f"{name} = {n} does not split over {world} ranks")
    hq, hk = n_heads // world, n_kv_heads // world
    q0 = rank * hq * head_dim
    k0 = n_heads * head_dim + rank * hk * head_dim
    v0 = (n_heads + n_kv_heads) * head_dim + rank * hk * head_dim
    f0, f1 = shard_rows(ffn, rank, world)
    return {
        "qkv": [(q0, q0 + hq * head_dim), (k0, k0 + hk * head_dim), (v0, v0 + hk * head_dim)],
        "o": [shard_rows(d_model, rank, world)],
        "gate_up": [(f0, f1), (ffn + f0, ffn + f1)],
        "down": [shard_rows(d_model, rank, world)],
        "lm_head": [shard_rows(vocab, rank, world)],
        "kv_heads": shard_rows(n_kv_heads, rank, world),
    }


def exchange_handles(local: bytes, rank: int, world: int, group=None) -> List[bytes]:
    """All-gather of the 64-byte IPC handles through torch.distributed (any backend)."""
    import torch.distributed as dist
    if world == 1:
        return [local]
    out: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(out, bytes(local), group=group)
    return [bytes(h) for h in out]


class Comm:
    """One rank's window plus its peers' (``rcu_comm``)."""

    def __init__(self, dev: Device, rank: int, world: int, max_out_elems: int, group=None, bytes_per_elem: int = 2):
        """Slots hold `max_out_elems` elements of `bytes_per_elem` bytes: 2 for the f16 outputs of
        ``linear``, 4 for a sharded ``Decoder`` (its exchanges carry one tagged word per element)."""
        self.dev, self.rank, self.world = dev, rank, world
        h = C.c_void_p()
        slot_bytes = (max_out_elems * bytes_per_elem + 15) // 16 * 16
        dev.check(dev._lib.rcu_comm_create(dev.handle, rank, world, slot_bytes, C.byref(h)))
        self._h = h
        handle = (C.c_ubyte * 64)()
        dev.check(dev._lib.rcu_comm_export(self._h, handle))
        handles = exchange_handles(bytes(handle), rank, world, group)
        for p, hb in enumerate(handles):
            if p == rank:
                continue
            arr = (C.c_ubyte * 64).from_buffer_copy(hb)
            dev.check(dev._lib.rcu_comm_import(self._h, p, arr))

    def close(self) -> None:
        if self._h is not None and self.dev.handle:
            self.dev._lib.rcu_comm_destroy(self._h)
        self._h = None

    def linear(self, w_shard: Buffer, x: Buffer, n_total: int, bias_shard: Optional[Buffer] = None) -> Buffer:
        """y[1, n_total] = all_gather_r(W_r . x): every rank gets the full f16 output (a view of the
        rank's window, valid until the call after next)."""
        y = C.c_void_p()
        self.dev.check(self.dev._lib.rcu_gemv_q8_allgather(self._h, C.byref(w_shard.desc()), C.byref(x.desc()),
                                                           C.byref(bias_shard.desc()) if bias_shard is not None else None,
                                                           C.byref(y)))
        return self.dev.wrap(capi.F16, (1, n_total), y.value)
