"""Decode attention without device allocation (``rcu_attn_decode_static``).

Some users of this library cannot allocate device memory at the point where they need attention:
a plug-in inside a host framework that owns the device heap, a serving loop that cannot afford the
device-wide synchronisation an allocation implies, a process that gave all free memory to its KV
caches.  For them the library carries the split-KV scratch inside its own device image.  This test
calls that entry point through the C ABI, twice in a row on different inputs (the built-in scratch
is shared and keeps the previous call's contents), and checks each result against the ordinary
entry point, which takes its scratch from the allocator.  The file name sorts last so that a run
that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(dev, fn, qkv, kc, vc, H, Hkv, hd, max_cache, rope_dim, P):
    from ratchet_b200 import capi
    dq, dk, dv = dev.from_numpy(qkv), dev.from_numpy(kc), dev.from_numpy(vc)
    out = dev.empty(capi.F16, (H * hd,))
    dev.check(fn(dev.handle, dq.ptr, dk.ptr, dv.ptr, H, Hkv, hd, max_cache, rope_dim, 10000.0, P, out.ptr))
    return out.to_numpy().astype(np.float32), dk.to_numpy(), dv.to_numpy()


def test_static_scratch_attention_matches_allocating_entry_point():
    from ratchet_b200 import Device, RatchetCudaError, capi
    dev = Device(0)
    try:
        lib = dev._lib
        # two calls in a row with different shapes, so stale scratch from the first would show in the second
        for (H, Hkv, hd, rope_dim, max_cache, P) in [(32, 32, 96, 96, 4096, 1024), (8, 2, 64, 32, 512, 300)]:
            g = np.random.Generator(np.random.PCG64(H + P))
            qkv = g.standard_normal((H + 2 * Hkv) * hd).astype(np.float16)
            kc = np.zeros((Hkv, max_cache, hd), np.float16)
            vc = np.zeros((Hkv, max_cache, hd), np.float16)
            kc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
            vc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
            got, k1, v1 = _run(dev, lib.rcu_attn_decode_static, qkv, kc, vc, H, Hkv, hd, max_cache, rope_dim, P)
            ref, k0, v0 = _run(dev, lib.rcu_attn_decode, qkv, kc, vc, H, Hkv, hd, max_cache, rope_dim, P)
            # same kernel, same inputs: within the 1e-2 bar of the other attention tests (in practice equal)
            scale = np.sqrt(np.mean(ref.astype(np.float64) ** 2)) + 1e-30
            assert np.abs(got - ref).max() / scale < 1e-2
            assert np.array_equal(k1.view(np.uint16), k0.view(np.uint16))
            assert np.array_equal(v1.view(np.uint16), v0.view(np.uint16))
        # beyond the built-in scratch: refused with a message that names the limit, nothing launched
        too_many = 65
        dq = dev.from_numpy(np.zeros(3 * too_many * 64, np.float16))
        dk = dev.from_numpy(np.zeros((too_many, 8, 64), np.float16))
        out = dev.empty(capi.F16, (too_many * 64,))
        with pytest.raises(RatchetCudaError) as e:
            dev.check(lib.rcu_attn_decode_static(dev.handle, dq.ptr, dk.ptr, dk.ptr, too_many, too_many, 64, 8, 64, 10000.0, 0, out.ptr))
        assert e.value.status == capi.ERR_INVALID_ARG and "at most 64 heads" in str(e.value)
    finally:
        dev.close()
