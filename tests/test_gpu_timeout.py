"""A device-side wait that runs out: the kernel gives up on its own, the next synchronisation reports
RCU_ERR_TIMEOUT, and the device stays usable.  The failure is made on the host: two exchange windows are
created on one device and linked to each other in-process, but only "rank 0" ever launches, so the
arrival counter its kernel waits for is never incremented.  Nothing faults or hangs; the wait limit is
20 ms for the test."""
import ctypes as C
import time

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_unanswered_exchange_times_out_and_the_device_stays_usable():
    from ratchet_b200 import Device, RatchetCudaError, capi
    dev = Device(0)
    lib = dev._lib
    c0, c1 = C.c_void_p(), C.c_void_p()
    try:
        N, K = 512, 2048
        dev.check(lib.rcu_comm_create(dev.handle, 0, 2, N * 2, C.byref(c0)))
        dev.check(lib.rcu_comm_create(dev.handle, 1, 2, N * 2, C.byref(c1)))
        dev.check(lib.rcu_comm_import_local(c0, 1, c1))
        dev.check(lib.rcu_comm_import_local(c1, 0, c0))
        g = np.random.Generator(np.random.PCG64(0))
        w = (g.standard_normal((N // 2, K)) * 0.02).astype(np.float16)
        x = g.standard_normal((1, K)).astype(np.float16)
        wq = orc.quantize_q8(w)
        dw = dev.from_quantized(wq, capi.Q8_0H, (N // 2, K))
        dx = dev.from_numpy(x)
        dev.set_wait_limit_ns(20_000_000)
        y = C.c_void_p()
        t0 = time.perf_counter()
        dev.check(lib.rcu_gemv_q8_allgather(c0, C.byref(dw.desc()), C.byref(dx.desc()), None, C.byref(y)))
        with pytest.raises(RatchetCudaError) as e:
            dev.sync()
        waited = time.perf_counter() - t0
        assert e.value.status == capi.ERR_TIMEOUT
        assert 0.015 < waited < 1.5, waited            # the kernel gave up after the limit, not after the two-second default
        # rank 0's own half of the output is complete and correct all the same
        half = np.empty(N // 2, np.float16)
        dev.d2h(half, y.value, N)
        ref = orc.gemv_q8(wq, N // 2, K, True, x.reshape(-1)).astype(np.float32)
        assert np.abs(half.astype(np.float32) - ref).max() / np.sqrt(np.mean(ref * ref)) < 1e-2
        # the flag was consumed by that sync: the device goes on working
        dev.set_wait_limit_ns(2_000_000_000)
        dev.sync()
        out = dev.matmul(dw, dx, None, False, True, True).to_numpy().astype(np.float32).reshape(-1)
        assert np.abs(out - ref).max() / np.sqrt(np.mean(ref * ref)) < 1e-2
    finally:
        if c0:
            lib.rcu_comm_destroy(c0)
        if c1:
            lib.rcu_comm_destroy(c1)
        dev.close()
