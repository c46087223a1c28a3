"""The library's Q8_0 quantiser (rcu_quantize on the host, rcu_quantize_device on the GPU) against the
oracle's restatement of ratchet-core/src/quant.rs:19-99: the buffers must agree bit for bit, including
the reference's corner cases."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc


def _cases(dtype):
    g = np.random.Generator(np.random.PCG64(5))
    w = (g.standard_normal((96, 512)) * 0.02).astype(dtype)
    edge = (g.standard_normal((8, 32))).astype(dtype)
    edge[0] = 0                          # d = 0: x / d is NaN, which Rust's `as i32` turns into 0
    edge[1, 3] = np.nan                  # max() ignores NaN; NaN / d -> 0
    edge[2, 5] = np.inf                  # d = inf: finite / inf = 0, inf / inf = NaN -> 0
    edge[3] = dtype(6e-8) if dtype is np.float16 else dtype(1e-44)   # subnormal maximum: d rounds to 0 in f16 -> x / 0 = inf -> saturates
    edge[4] = np.finfo(dtype).max
    edge[5, ::2] *= -1
    edge[6] = dtype(-0.0)
    tie = np.zeros((1, 32), dtype)       # ratios of exactly k + 0.5 round away from zero
    tie[0, 0] = 127
    tie[0, 1:9] = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5, -63.5], dtype)
    return [w, edge, tie, (g.standard_normal((1, 32)) * 100).astype(dtype)]


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_host_quantiser_is_bit_exact(dtype):
    from ratchet_b200 import capi
    for x in _cases(dtype):
        with np.errstate(all="ignore"):
            got = capi.quantize(x)
        ref = orc.quantize_q8(x)
        assert got.shape == ref.shape
        assert np.array_equal(got, ref), f"{dtype.__name__} {x.shape}: {np.flatnonzero(got != ref)[:8]}"


def test_host_quantiser_round_trip_and_errors():
    from ratchet_b200 import capi
    g = np.random.Generator(np.random.PCG64(9))
    # 256 KiB of blocks: the threaded path
    x = (g.standard_normal((512, 4096)) * 0.02).astype(np.float32)
    buf = capi.quantize(x)
    assert np.array_equal(buf, orc.quantize_q8(x))
    back = orc.dequantize_q8(buf, x.shape, False)
    assert np.abs(back - x).max() <= np.abs(x).reshape(-1, 32).max(1).max() / 127 * 0.5001   # test_quantization_reflexivity's bound
    lib = capi.lib()
    out = np.empty(64, np.uint8)
    src = np.zeros(33, np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    assert lib.rcu_quantize(capi.Q8_0F, p(src), 33, p(out), 64) == capi.ERR_INVALID_ARG        # not whole blocks
    assert lib.rcu_quantize(capi.Q8_0F, p(src), 32, p(out), 64) == capi.ERR_INVALID_ARG        # output too small (512 needed)
    assert lib.rcu_quantize(capi.Q4_KF, p(src), 32, p(out), 64) == capi.ERR_UNSUPPORTED
    assert lib.rcu_quantize(capi.F32, p(src), 32, p(out), 64) == capi.ERR_UNSUPPORTED


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_device_quantiser_is_bit_exact(dtype):
    from ratchet_b200 import Device, capi
    dev = Device(0)
    try:
        for x in _cases(dtype) + [(np.random.Generator(np.random.PCG64(2)).standard_normal((3072, 3072)) * 0.02).astype(dtype)]:
            got = dev.quantize(dev.from_numpy(x))
            assert got.dt == (capi.Q8_0H if dtype is np.float16 else capi.Q8_0F) and got.shape == x.shape
            ref = orc.quantize_q8(x)
            assert np.array_equal(got.to_numpy(), ref), f"{dtype.__name__} {x.shape}"
            if not np.isfinite(x.astype(np.float32)).all() or np.abs(x.astype(np.float32)).max() > 1e4:
                continue                # NaN payloads of a dequantised inf * 0 are not pinned
            # and it is a valid operand: dequantise on the device gives the oracle's dequantisation
            dq = dev.dequantize(got).to_numpy()
            exp = orc.dequantize_q8(ref, x.shape, dtype is np.float16)
            assert np.array_equal(dq.view(np.uint16 if dtype is np.float16 else np.uint32), exp.view(np.uint16 if dtype is np.float16 else np.uint32))
    finally:
        dev.close()
