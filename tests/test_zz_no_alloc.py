"""Decode attention without device allocation (``rcu_attn_decode_static``).

Some users of this library cannot allocate device memory at the point where they need attention:
a plug-in inside a host framework that owns the device heap, a serving loop that cannot afford the
device-wide synchronisation an allocation implies, a process that gave all free memory to its KV
caches.  For them the library carries the split-KV scratch inside its own device image.  This test
calls that entry point through the C ABI, several times in a row on different inputs (the built-in
scratch is shared and keeps the previous call's contents), and checks each result against the
ordinary entry point, which takes its scratch from the allocator, and against the float64
restatement of the reference's attention graph.  Cached lengths beyond 2048 positions take the
split-KV kernel, which is the one that writes per-tile partial results and per-head completion
counters into the built-in array; shorter ones take the cluster kernel, which reads only the RoPE
table and the position word from it.  The file name sorts last so that a run that stops at the first
failure has already run every other test.
"""
import numpy as np
import pytest

from .test_gpu_decode import attention_reference, rel_err

pytestmark = pytest.mark.gpu


def _run(dev, fn, qkv, kc, vc, H, Hkv, hd, max_cache, rope_dim, P):
    from ratchet_b200 import capi
    dq, dk, dv = dev.from_numpy(qkv), dev.from_numpy(kc), dev.from_numpy(vc)
    out = dev.empty(capi.F16, (H * hd,))
    dev.check(fn(dev.handle, dq.ptr, dk.ptr, dv.ptr, H, Hkv, hd, max_cache, rope_dim, 10000.0, P, out.ptr))
    res = out.to_numpy().astype(np.float32), dk.to_numpy(), dv.to_numpy()
    for t in (dq, dk, dv, out):
        t.free()
    return res


# (H, Hkv, hd, rope_dim, max_cache, P), run in this order on one device: a large split-KV case is followed by a
# smaller one so that partial results left by the first lie where the second would read them if it read
# too far; then the largest shape the built-in array holds; then the cluster-kernel cases.
CASES = [(32, 32, 96, 96, 4096, 3000), (8, 2, 64, 32, 4096, 2500), (64, 64, 128, 128, 4096, 4095), (32, 32, 96, 96, 4096, 1024),
         (8, 2, 64, 32, 512, 300)]


def test_static_scratch_attention_matches_allocating_entry_point():
    from ratchet_b200 import Device, RatchetCudaError, capi
    dev = Device(0)
    try:
        lib = dev._lib
        for (H, Hkv, hd, rope_dim, max_cache, P) in CASES:
            g = np.random.Generator(np.random.PCG64(H + P))
            qkv = g.standard_normal((H + 2 * Hkv) * hd).astype(np.float16)
            kc = np.zeros((Hkv, max_cache, hd), np.float16)
            vc = np.zeros((Hkv, max_cache, hd), np.float16)
            kc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
            vc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
            got, k1, v1 = _run(dev, lib.rcu_attn_decode_static, qkv, kc, vc, H, Hkv, hd, max_cache, rope_dim, P)
            ref, k0, v0 = _run(dev, lib.rcu_attn_decode, qkv, kc, vc, H, Hkv, hd, max_cache, rope_dim, P)
            what = f"H={H} hd={hd} P={P}"
            # same kernel, same inputs: within the 1e-2 bar of the other attention tests (in practice equal)
            assert rel_err(got, ref) < 1e-2, what
            assert np.array_equal(k1.view(np.uint16), k0.view(np.uint16)), what
            assert np.array_equal(v1.view(np.uint16), v0.view(np.uint16)), what
            # and against the reference's attention graph restated in float64 (it appends to kc / vc)
            cpu = attention_reference(qkv, kc, vc, H, Hkv, hd, rope_dim, 10000.0, P)
            assert rel_err(got, cpu) < 1e-2, what
        # beyond the built-in scratch: refused with a message that names the limit, nothing launched
        too_many = 65
        dq = dev.from_numpy(np.zeros(3 * too_many * 64, np.float16))
        dk = dev.from_numpy(np.zeros((too_many, 8, 64), np.float16))
        out = dev.empty(capi.F16, (too_many * 64,))
        with pytest.raises(RatchetCudaError) as e:
            dev.check(lib.rcu_attn_decode_static(dev.handle, dq.ptr, dk.ptr, dk.ptr, too_many, too_many, 64, 8, 64, 10000.0, 0, out.ptr))
        assert e.value.status == capi.ERR_INVALID_ARG and "at most 64 heads" in str(e.value)
        with pytest.raises(RatchetCudaError) as e:
            dev.check(lib.rcu_attn_decode_static(dev.handle, dq.ptr, dk.ptr, dk.ptr, 8, 8, 64, 4097, 64, 10000.0, 0, out.ptr))
        assert e.value.status == capi.ERR_INVALID_ARG and "at most 4096 positions" in str(e.value)
    finally:
        dev.close()
