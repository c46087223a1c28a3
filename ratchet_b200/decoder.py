"""Fused decode step: the per-token graph of ``Phi3::schedule``
(crates/ratchet-models/src/phi3/model.rs:134-156) as one CUDA-graph replay of fused kernels.

``Decoder`` takes the same tensors the lazy model holds (Q8_0 Linear weights, f32 RMSNorm scales, the
f16 KV caches of ratchet-nn's ``KVCache``) as device ``Buffer`` objects and runs
``rcu_decoder_step`` per token.  It is the product path the benchmark times for the Phi-3-mini
decode configuration; the lazy ``Tensor`` graph of ``ratchet_b200.callers.Phi3`` computes the same
function node by node and is what the parity tests compare it with.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from . import capi
from .capi import RatchetCudaError
from .device import Buffer, Device


@dataclass
class DecoderConfig:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    max_cache: int = 4096          # Phi3::MAX_CACHE (phi3/model.rs:160)
    rope_dim: int = 96
    rope_base: float = 10000.0
    rms_eps: float = 1e-5
    weight_dt: int = capi.Q8_0H


@dataclass
class DecoderLayer:
    attn_norm: Buffer
    qkv: Buffer
    o: Buffer
    ffn_norm: Buffer
    gate_up: Buffer
    down: Buffer
    k_cache: Buffer
    v_cache: Buffer


class Decoder:
    """``comm`` = None: the whole model on one GPU.  With a ``ratchet_b200.comm.Comm`` the step is sharded
    over the comm's ranks (one process per GPU): ``cfg`` still describes the whole model, ``layers`` and
    ``lm_head`` hold this rank's rows (``comm.decoder_shard_ranges``), the KV caches its own heads; the
    comm must be fresh, with slots of ``max(d_model, ffn, vocab, n_heads * head_dim)`` elements of 4 bytes
    (``Comm(..., bytes_per_elem=4)``), and every rank must step with the same token."""

    def __init__(self, dev: Device, cfg: DecoderConfig, layers: List[DecoderLayer], tok_embd: Buffer, out_norm: Buffer,
                 lm_head: Buffer, comm=None):
        self.dev, self.cfg = dev, cfg
        self._keep = (layers, tok_embd, out_norm, lm_head, comm)     # device memory must outlive the decoder
        c = capi.rcu_decoder_config(cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab,
                                    cfg.max_cache, cfg.rope_dim, cfg.rope_base, cfg.rms_eps, cfg.weight_dt)
        arr = (capi.rcu_decoder_layer * len(layers))()
        for i, l in enumerate(layers):
            arr[i] = capi.rcu_decoder_layer(l.attn_norm.ptr, l.qkv.ptr, l.o.ptr, l.ffn_norm.ptr, l.gate_up.ptr, l.down.ptr,
                                            l.k_cache.ptr, l.v_cache.ptr)
        h = C.c_void_p()
        if comm is None:
            dev.check(dev._lib.rcu_decoder_create(dev.handle, C.byref(c), arr, tok_embd.ptr, out_norm.ptr, lm_head.ptr, C.byref(h)))
        else:
            dev.check(dev._lib.rcu_decoder_create_sharded(dev.handle, comm._h, C.byref(c), arr, tok_embd.ptr, out_norm.ptr, lm_head.ptr,
                                                          C.byref(h)))
        self._h = h
        self.token = dev.empty(capi.I32, (1,))
        self.logits = dev.empty(capi.F16, (1, 1, cfg.vocab))
        self.next_token = dev.empty(capi.I32, (1,))

    def close(self) -> None:
        if self._h is not None and self.dev.handle:
            self.dev._lib.rcu_decoder_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def position(self) -> int:
        return self.dev._lib.rcu_decoder_position(self._h)

    @position.setter
    def position(self, p: int) -> None:
        self.dev.check(self.dev._lib.rcu_decoder_set_position(self._h, p))

    @property
    def kernels_per_step(self) -> int:
        return self.dev._lib.rcu_decoder_kernels_per_step(self._h)

    def step_device(self, token_ptr: Optional[int] = None, argmax: bool = True) -> None:
        """One step entirely on the device: token id read from device memory, logits and (optionally)
        the arg-max id written to device memory.  Asynchronous."""
        tp = self.token.ptr if token_ptr is None else token_ptr
        self.dev.check(self.dev._lib.rcu_decoder_step(self._h, C.c_void_p(tp), C.c_void_p(self.logits.ptr),
                                                      C.c_void_p(self.next_token.ptr) if argmax else None))

    def profile_step(self, token_ptr: Optional[int] = None) -> np.ndarray:
        """One step outside the CUDA graph with time stamps of the data-flow kernel's first CTA (device
        nanoseconds): for every job — per layer qkv, attention, o, gate/up, down, then lm_head — when it began
        and when its input was staged; then the kernel's end; then 6 x 4 cycle sums of the grid's first warp (per job
        kind: slot wait, multiply, store, request)."""
        tp = self.token.ptr if token_ptr is None else token_ptr
        cap = 2 * (5 * self.cfg.n_layers + 1) + 1 + 24
        stamps = np.zeros(cap, np.uint64)
        n = C.c_uint32()
        self.dev.check(self.dev._lib.rcu_decoder_profile_step(self._h, C.c_void_p(tp), C.c_void_p(self.logits.ptr),
                                                              stamps.ctypes.data_as(C.POINTER(C.c_uint64)), cap, C.byref(n)))
        return stamps[: n.value]

    def step(self, token_id: int) -> np.ndarray:
        """What one iteration of the reference's generate loop does (phi3/generate.rs:93-113): upload the
        token id, run the model, bring the logits back to the host (f16 [1,1,vocab])."""
        self.dev.h2d(self.token.ptr, np.array([token_id], np.int32))
        self.step_device(argmax=False)
        return self.logits.to_numpy()
