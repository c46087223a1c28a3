"""Parity of every CUDA op with the CPU oracle, through the C ABI, on identical seeded inputs.

Bars: dequantisation / indexing / copies bit-exact; f32 ops within 1e-4
(relative, with an equal absolute floor as in the reference's all_close, tensor.rs:1039-1043);
f16 and quantised matmuls within 1e-2.
"""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from ratchet_b200 import Device
    d = Device(0)
    yield d
    d.close()


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def assert_close(a, b, tol, what=""):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    same_inf = np.isinf(a) & np.isinf(b) & (np.sign(a) == np.sign(b))   # e.g. exp overflow in f16 on both sides
    with np.errstate(invalid="ignore"):
        bad = ~same_inf & ~(np.abs(a - b) <= tol + tol * np.abs(b))
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tol {tol}; max abs err {np.nanmax(np.abs(a - b)[~same_inf]):.3e}"


def assert_matmul_close(a, b, tol, what=""):
    # relative to the result's scale: |a-b| <= tol * (rms(b) + |b|)
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    scale = np.sqrt(np.mean(b * b)) + 1e-30
    bad = np.abs(a - b) > tol * (scale + np.abs(b))
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside {tol}; max abs {np.abs(a - b).max():.3e}, rms {scale:.3e}"


def bits(a):
    return a.view(np.uint16 if a.itemsize == 2 else np.uint32)


# ------------------------------------------------------------------------------ quantised layouts
@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("shape", [(1, 32), (7, 96), (64, 3072), (33, 4096)])
def test_dequantize_q8_bit_exact(dev, half, shape):
    from ratchet_b200 import capi
    x = (rng(1).standard_normal(shape) * 0.02).astype(np.float16 if half else np.float32)
    buf = orc.quantize_q8(x)
    buf[0] = 0x80  # -128 never comes out of the quantiser but can come out of a GGUF file
    d = dev.from_quantized(buf, capi.Q8_0H if half else capi.Q8_0F, shape)
    got = dev.dequantize(d).to_numpy()
    assert np.array_equal(bits(got), bits(orc.dequantize_q8(buf, shape, half)))


@pytest.mark.parametrize("half", [False, True])
def test_dequantize_q4k_bit_exact(dev, half):
    from ratchet_b200 import capi
    shape = (24, 512)
    x = (rng(2).standard_normal(shape) * 0.02).astype(np.float32)
    buf = orc.quantize_q4k(x, half)
    d = dev.from_quantized(buf, capi.Q4_KH if half else capi.Q4_KF, shape)
    got = dev.dequantize(d).to_numpy()
    assert np.array_equal(bits(got), bits(orc.dequantize_q4k(buf, shape, half)))


def test_layout_queries_match_oracle():
    from ratchet_b200 import capi
    for n in (32 * 7, 256 * 3, 3072 * 3072):
        assert capi.dtype_nbytes(capi.Q8_0F, n) == orc.q8_nbytes(n, False)
        assert capi.dtype_nbytes(capi.Q8_0H, n) == orc.q8_nbytes(n, True)
        assert capi.dtype_segments(capi.Q8_0H, n)[1] == orc.q8_scale_offset(n)
    for n in (256 * 3, 8192 * 3072):
        for half in (False, True):
            dt = capi.Q4_KH if half else capi.Q4_KF
            assert capi.dtype_nbytes(dt, n) == orc.q4k_nbytes(n, half)
            assert capi.dtype_segments(dt, n) == orc.q4k_offsets(n, half)


# ------------------------------------------------------------------------------ GEMV (decode)
GEMV_SHAPES = [(1, 32), (5, 64), (33, 480), (256, 512), (1000, 544), (3072, 3072), (3071, 1024), (512, 8192), (40, 16384)]


@pytest.mark.parametrize("pair", ["Q8_0F/F32", "Q8_0H/F16", "Q8_0F/F16"])
@pytest.mark.parametrize("N,K", GEMV_SHAPES)
def test_gemv_q8(dev, pair, N, K):
    from ratchet_b200 import capi
    g = rng(N * 131 + K)
    half_w = pair.startswith("Q8_0H")
    half_x = pair.endswith("F16")
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float16 if half_w else np.float32)
    x = g.standard_normal((1, K)).astype(np.float16 if half_x else np.float32)
    bias = g.standard_normal(N).astype(x.dtype)
    wq = orc.quantize_q8(w)
    for b in (None, bias):
        ref = orc.gemv_q8(wq, N, K, half_w, x.reshape(-1), b)
        dw = dev.from_quantized(wq, capi.Q8_0H if half_w else capi.Q8_0F, (N, K))
        # Linear convention (ratchet-nn/src/linear.rs:17-24)
        y = dev.matmul(dw, dev.from_numpy(x), None if b is None else dev.from_numpy(b), False, True, True)
        assert y.shape == (1, N) and y.dt == (capi.F16 if half_x else capi.F32)
        assert_matmul_close(y.to_numpy().reshape(-1), ref, 1e-2 if half_x else 1e-4, f"gemv {pair} {N}x{K}")


def test_gemv_back_to_back_with_constant_weights(dev):
    """The caller's promise that its weights are not being written (rcu_set_constant_weights) lets consecutive
    GEMVs overlap: each is launched as a programmatic dependent and asks for weight rows before its predecessor
    has ended, while activations and outputs still wait for it.  A chain y1 = W1 x, y2 = W2 y1, y3 = W3 y2 launched
    without any synchronisation in between must give what the same chain gives without the promise."""
    from ratchet_b200 import capi
    g = rng(99)
    K = 3072
    ws = [orc.quantize_q8((g.standard_normal((K, K)) * 0.02).astype(np.float16)) for _ in range(3)]
    dws = [dev.from_quantized(w, capi.Q8_0H, (K, K)) for w in ws]
    x = dev.from_numpy(g.standard_normal((1, K)).astype(np.float16))

    def chain():
        h = x
        for dw in dws:
            h = dev.matmul(dw, h, None, False, True, True)
        return h.to_numpy()

    base = chain()
    dev.set_constant_weights(True)
    try:
        for _ in range(3):
            assert np.array_equal(chain().view(np.uint16), base.view(np.uint16))
    finally:
        dev.set_constant_weights(False)
    h = x.to_numpy().reshape(-1)
    for w in ws:
        h = orc.gemv_q8(w, K, K, True, h).astype(np.float16)
    assert_matmul_close(base.reshape(-1), h, 2e-2, "chain of three GEMVs")


def test_gemv_q8_headline_shape(dev):
    """The benchmark's shape, K = 16384 x N = 65536 with f32 block scales and f16 activations (1.2 GB of
    weights: the plain streaming kernel with its K split of 8).  The matrix is 4096 distinct random rows
    repeated down the 65536, as the benchmark builds it; the oracle computes the distinct rows once and
    every repetition on the device must reproduce them."""
    from ratchet_b200 import capi
    K, N, uniq = 16384, 65536, 4096
    g = rng(65536)
    w = (g.standard_normal((uniq, K), dtype=np.float32) * np.float32(0.02))
    x = g.standard_normal((1, K)).astype(np.float16)
    small = orc.quantize_q8(w)
    ref = orc.gemv_q8(small, uniq, K, False, x.reshape(-1))
    buf = np.zeros(capi.dtype_nbytes(capi.Q8_0F, N * K), np.uint8)
    off_small = capi.dtype_segments(capi.Q8_0F, uniq * K)[1]
    off = capi.dtype_segments(capi.Q8_0F, N * K)[1]
    buf[: N * K].reshape(N // uniq, uniq * K)[:] = small[: uniq * K]
    buf[off: off + N * K // 8].reshape(N // uniq, uniq * K // 8)[:] = small[off_small: off_small + uniq * K // 8]
    dw = dev.from_quantized(buf, capi.Q8_0F, (N, K))
    del buf
    y = dev.matmul(dw, dev.from_numpy(x), None, False, True, True).to_numpy().reshape(N // uniq, uniq)
    dw.free()
    for rep in range(N // uniq):
        assert_matmul_close(y[rep], ref, 1e-2, f"headline gemv, rows {rep * uniq}..")
    # every repetition of a row is computed by a different warp team but from the same bytes
    assert np.array_equal(bits(np.ascontiguousarray(y[0])), bits(np.ascontiguousarray(y[-1])))


@pytest.mark.parametrize("pair", ["Q8_0H/F16", "Q8_0F/F16"])
@pytest.mark.parametrize("N,K", [(512, 8192), (3072, 3072), (40, 16384)])
@pytest.mark.parametrize("kind", ["one_large", "one_percent_x50", "huge"])
def test_gemv_q8_activation_outliers(dev, pair, N, K, kind):
    """Activation vectors with outliers, as transformer residual streams have them: the f16-activation
    kernels re-express x in 16-bit fixed point per group of 16 elements, so a large element must not cost
    the others their precision.  Bar as for every f16 matmul: 1e-2 of the result's scale."""
    from ratchet_b200 import capi
    g = rng(N + K + len(kind))
    half_w = pair.startswith("Q8_0H")
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float16 if half_w else np.float32)
    x = g.standard_normal(K).astype(np.float32)
    if kind == "one_large":
        x[K // 3] = 200.0
    elif kind == "one_percent_x50":
        x[g.choice(K, K // 100, replace=False)] *= 50.0
    else:
        # 1e3 times the typical magnitude, meeting zero weights: the result is made of the ordinary elements
        # alone, so any precision they lost to the outlier shows at the result's own scale (with one scale for
        # the whole vector every other element would be rounded to a multiple of 0.03)
        x[7] = 1000.0
        w[:, 7] = 0
    x = x.astype(np.float16).reshape(1, K)
    wq = orc.quantize_q8(w)
    ref = orc.gemv_q8(wq, N, K, half_w, x.reshape(-1))
    dw = dev.from_quantized(wq, capi.Q8_0H if half_w else capi.Q8_0F, (N, K))
    y = dev.matmul(dw, dev.from_numpy(x), None, False, True, True).to_numpy().reshape(-1)
    assert_matmul_close(y, ref, 1e-2, f"gemv outliers {kind} {pair} {N}x{K}")


@pytest.mark.parametrize("N,K", [(64, 512), (3072, 3072), (40, 16384)])
def test_gemv_q8_nan_activation_propagates(dev, N, K):
    """A NaN in x makes every output NaN, as it does in the reference's float arithmetic (each row's sum
    includes that element); an infinity makes every output non-finite."""
    from ratchet_b200 import capi
    g = rng(N ^ K)
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float16)
    wq = orc.quantize_q8(w)
    dw = dev.from_quantized(wq, capi.Q8_0H, (N, K))
    for bad in (np.nan, np.inf):
        x = g.standard_normal((1, K)).astype(np.float16)
        x[0, K // 2 + 1] = bad
        y = dev.matmul(dw, dev.from_numpy(x), None, False, True, True).to_numpy().reshape(-1)
        ref = orc.gemv_q8(wq, N, K, True, x.reshape(-1))
        assert not np.isfinite(ref).any()
        assert not np.isfinite(y.astype(np.float32)).any()
        if np.isnan(bad):
            assert np.isnan(y.astype(np.float32)).all()


# Q4_K weights with a vector: no kernel in the reference (`(gemv, q4)` is todo!, ops/matmul/mod.rs:746); the
# meaning is the dequantised product, as for every quantised op
@pytest.mark.parametrize("pair", ["Q4_KF/F32", "Q4_KH/F16"])
@pytest.mark.parametrize("N,K", [(1, 256), (5, 512), (33, 768), (1000, 1024), (3072, 3072), (3071, 1280), (8192, 3072), (40, 16384)])
def test_gemv_q4k(dev, pair, N, K):
    from ratchet_b200 import capi
    g = rng(N * 17 + K)
    half = pair.startswith("Q4_KH")
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = g.standard_normal((1, K)).astype(np.float16 if half else np.float32)
    bias = g.standard_normal(N).astype(x.dtype)
    buf = orc.quantize_q4k(w, half)
    wd = orc.dequantize_q4k(buf, (N, K), half)
    dw = dev.from_quantized(buf, capi.Q4_KH if half else capi.Q4_KF, (N, K))
    for b in (None, bias):
        ref = orc.matmul(wd, x, b, False, True, True)
        y = dev.matmul(dw, dev.from_numpy(x), None if b is None else dev.from_numpy(b), False, True, True)
        assert y.shape == (1, N) and y.dt == (capi.F16 if half else capi.F32)
        assert_matmul_close(y.to_numpy(), ref, 1e-2 if half else 1e-4, f"gemv {pair} {N}x{K}")
    # a zero vector gives the bias (the activation scale is guarded)
    y0 = dev.matmul(dw, dev.from_numpy(np.zeros_like(x)), dev.from_numpy(bias), False, True, True)
    assert np.array_equal(y0.to_numpy().reshape(-1), bias)


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("N,K", [(1, 1), (3, 7), (64, 100), (500, 1024), (3072, 3072), (96, 1025)])
def test_gemv_float(dev, dt, N, K):
    g = rng(N * 7 + K)
    T = np.float32 if dt == "f32" else np.float16
    w = g.standard_normal((N, K)).astype(T)
    x = g.standard_normal((K, 1)).astype(T)
    ref = orc.matmul(w, x)
    y = dev.matmul(dev.from_numpy(w), dev.from_numpy(x))
    assert y.shape == (N, 1)
    assert_matmul_close(y.to_numpy(), ref, 1e-4 if dt == "f32" else 1e-2, f"gemv {dt} {N}x{K}")


# ------------------------------------------------------------------------------ GEMM (general)
TRANS = [(False, False, False), (True, False, False), (False, True, False), (False, False, True), (True, True, False), (False, True, True)]


@pytest.mark.parametrize("tl,tr,td", TRANS)
@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_gemm_vs_oracle(dev, tl, tr, td, dt):
    # shape distribution of the reference's matmul tests: B 1..3, M,K,N 1..256 (ops/matmul/mod.rs:818-853)
    g = rng(100 + tl * 4 + tr * 2 + td + (8 if dt == "f16" else 0))
    T = np.float32 if dt == "f32" else np.float16
    for _ in range(5):
        B, M, K, N = (int(v) for v in (g.integers(1, 4), g.integers(1, 257), g.integers(1, 257), g.integers(2, 257)))
        a = g.standard_normal((B, K, M) if tl else (B, M, K)).astype(T)
        b = g.standard_normal((B, N, K) if tr else (B, K, N)).astype(T)
        ref = orc.matmul(a, b, None, tl, tr, td)
        y = dev.matmul(dev.from_numpy(a), dev.from_numpy(b), None, tl, tr, td)
        assert y.shape == ref.shape
        assert_matmul_close(y.to_numpy(), ref, 1e-4 if dt == "f32" else 1e-2, f"gemm {dt} {(B, M, K, N)}")


def test_gemm_stack_broadcast_and_bias(dev):
    g = rng(77)
    w = g.standard_normal((48, 40)).astype(np.float32)
    x = g.standard_normal((2, 3, 5, 40)).astype(np.float32)
    b = g.standard_normal(48).astype(np.float32)
    ref = orc.matmul(w, x, b, False, True, True)
    y = dev.matmul(dev.from_numpy(w), dev.from_numpy(x), dev.from_numpy(b), False, True, True)
    assert y.shape == (2, 3, 5, 48)
    assert_matmul_close(y.to_numpy(), ref, 1e-4)
    # attention-shaped batched products (phi3/attn.rs:142-157)
    q = g.standard_normal((1, 4, 1, 96)).astype(np.float32)
    k = g.standard_normal((1, 4, 33, 96)).astype(np.float32)
    ref = orc.matmul(q, k, None, False, True, False)
    y = dev.matmul(dev.from_numpy(q), dev.from_numpy(k), None, False, True, False)
    assert y.shape == (1, 4, 1, 33)
    assert_matmul_close(y.to_numpy(), ref, 1e-4)


@pytest.mark.parametrize("pair", ["Q8_0F/F32", "Q8_0H/F16", "Q4_KF/F32", "Q4_KH/F16"])
def test_gemm_quantised_weights(dev, pair):
    from ratchet_b200 import capi
    g = rng(5)
    N, K, M = 96, 512, 37
    half = pair.endswith("F16")
    T = np.float16 if half else np.float32
    w = (g.standard_normal((N, K)) * 0.02)
    x = g.standard_normal((2, M, K)).astype(T)
    if pair.startswith("Q8"):
        buf = orc.quantize_q8(w.astype(T))
        wd = orc.dequantize_q8(buf, (N, K), half)
        dt = capi.Q8_0H if half else capi.Q8_0F
    else:
        buf = orc.quantize_q4k(w.astype(np.float32), half)
        wd = orc.dequantize_q4k(buf, (N, K), half)
        dt = capi.Q4_KH if half else capi.Q4_KF
    ref = orc.matmul(wd, x, None, False, True, True)
    y = dev.matmul(dev.from_quantized(buf, dt, (N, K)), dev.from_numpy(x), None, False, True, True)
    assert y.shape == (2, M, N)
    assert_matmul_close(y.to_numpy(), ref, 1e-2 if half else 1e-4, pair)


def test_matmul_errors(dev):
    from ratchet_b200 import RatchetCudaError, capi
    a = dev.from_numpy(np.zeros((4, 5), np.float32))
    b = dev.from_numpy(np.zeros((6, 7), np.float32))
    with pytest.raises(RatchetCudaError) as e:
        dev.matmul(a, b)
    assert e.value.status == capi.ERR_INVALID_ARG
    h = dev.from_numpy(np.zeros((5, 7), np.float16))
    with pytest.raises(RatchetCudaError):
        dev.matmul(a, h, out=dev.empty(capi.F16, (4, 7)))   # (F32, F16) is not an allowed pair


# ------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary(dev, dt, op):
    g = rng(3)
    T = np.float32 if dt == "f32" else np.float16
    for shape in [(1,), (5,), (2, 33, 17), (1, 1, 3072), (3, 128, 130)]:
        a = g.standard_normal(shape).astype(T)
        b = (g.standard_normal(shape) + 3).astype(T)
        got = dev.binary(op, dev.from_numpy(a), dev.from_numpy(b)).to_numpy()
        assert np.array_equal(bits(got), bits(orc.binary(op, a, b))), f"{op} {dt} {shape}"


def test_binary_broadcast_and_inplace(dev):
    g = rng(4)
    a = g.standard_normal((1, 6, 50, 51)).astype(np.float32)
    for bshape in [(1,), (51,), (1, 6, 1, 1), (50, 1), (1, 1, 50, 51)]:
        b = g.standard_normal(bshape).astype(np.float32)
        ref = orc.binary("mul", a, np.ascontiguousarray(np.broadcast_to(b, a.shape)))
        got = dev.binary("mul", dev.from_numpy(a), dev.from_numpy(b)).to_numpy()
        assert np.array_equal(bits(got), bits(ref)), bshape
    # the left operand may be the broadcast one (tensor.rs:266-268)
    b = g.standard_normal((50, 51)).astype(np.float32)
    got = dev.binary("sub", dev.from_numpy(b), dev.from_numpy(a)).to_numpy()
    assert np.array_equal(bits(got), bits(orc.binary("sub", np.ascontiguousarray(np.broadcast_to(b, a.shape)), a)))
    da = dev.from_numpy(a)
    db = dev.from_numpy(a[::-1].copy())
    dev.binary("add", da, db, out=da)   # in place (ops/binary.rs:130-132)
    assert np.array_equal(bits(da.to_numpy()), bits(orc.binary("add", a, a[::-1].copy())))


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("op", list(orc.UNARY_OPS))
def test_unary(dev, dt, op):
    g = rng(6)
    T = np.float32 if dt == "f32" else np.float16
    x = g.standard_normal((2, 128, 65)).astype(T)
    x.reshape(-1)[:4] = [0.0, -0.0, 11.5, -11.5]   # beyond the WGSL tanh clamp (ops/unary.rs:187-195)
    if op in ("log", "sqrt"):
        x = (np.abs(x) + T(1e-3)).astype(T)
    ref = orc.unary(op, x)
    got = dev.unary(op, dev.from_numpy(x)).to_numpy()
    if op in ("abs", "relu", "floor", "ceil", "neg"):
        assert np.array_equal(bits(got), bits(ref))
    else:
        assert_close(got, ref, 1e-4 if dt == "f32" else 2e-3, f"{op} {dt}")


def test_cast(dev):
    from ratchet_b200 import capi
    x = rng(7).standard_normal((3, 1001)).astype(np.float32)
    x[0, :3] = [65520.0, 1e-8, -7.0e-5]   # f16 overflow, underflow, subnormal
    dx = dev.from_numpy(x)
    h = dev.cast(dx, capi.F16)
    assert np.array_equal(bits(h.to_numpy()), bits(orc.cast(x, orc.F32, orc.F16)))
    assert np.array_equal(bits(dev.cast(h, capi.F32).to_numpy()), bits(orc.cast(h.to_numpy(), orc.F16, orc.F32)))
    b = dev.cast(dx, capi.BF16)
    assert np.array_equal(b.to_numpy(), orc.cast(x, orc.F32, orc.BF16))
    assert np.array_equal(bits(dev.cast(b, capi.F32).to_numpy()), bits(orc.cast(b.to_numpy(), orc.BF16, orc.F32)))
    assert np.array_equal(dev.cast(dx, capi.I32).to_numpy(), x.view(np.int32))   # bit reinterpretation
    assert np.array_equal(dev.cast(dx, capi.U32).to_numpy(), x.view(np.uint32))


# ------------------------------------------------------------------------------ norm / softmax / reduce / rope
NORM_SHAPES = [(1, 1, 1), (2, 3, 7), (1, 64, 2560), (1, 150, 384), (1, 1, 3072), (3, 5, 1025), (1, 2, 9000)]


@pytest.mark.parametrize("shape", NORM_SHAPES)
@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_norms(dev, shape, dt):
    from ratchet_b200 import capi
    g = rng(8)
    T = np.float32 if dt == "f32" else np.float16
    tol = 1e-4 if dt == "f32" else 1e-2
    N = shape[-1]
    x = (g.standard_normal(shape) * 2 + 0.5).astype(T)
    s = g.standard_normal(N).astype(T)
    b = g.standard_normal(N).astype(T)
    dx, ds, db = dev.from_numpy(x), dev.from_numpy(s), dev.from_numpy(b)
    if N > 1:  # a single-element row has zero variance: rsqrt(eps) amplifies rounding
        assert_close(dev.norm(capi.LAYER_NORM, dx, ds, db, 1e-5).to_numpy(), orc.layer_norm(x, s, b, 1e-5), tol, "ln+bias")
        assert_close(dev.norm(capi.LAYER_NORM, dx, ds, None, 1e-5).to_numpy(), orc.layer_norm(x, s, None, 1e-5), tol, "ln")
    assert_close(dev.norm(capi.RMS_NORM, dx, ds, None, 1e-5).to_numpy(), orc.rms_norm(x, s, 1e-5), tol, "rms")


def test_group_norm_vs_torch(dev):
    import torch
    from ratchet_b200 import capi
    g = rng(9)
    x = g.standard_normal((2, 12, 50)).astype(np.float32)
    s = g.standard_normal(12).astype(np.float32)
    b = g.standard_normal(12).astype(np.float32)
    ref = torch.nn.functional.group_norm(torch.from_numpy(x), 3, torch.from_numpy(s), torch.from_numpy(b), 1e-5).numpy()
    got = dev.norm(capi.GROUP_NORM, dev.from_numpy(x), dev.from_numpy(s), dev.from_numpy(b), 1e-5, groups=3).to_numpy()
    assert_close(got, ref, 1e-4)


@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (2, 3, 7, 5), (1, 6, 150, 1500), (1, 32, 1, 1025), (2, 2, 3, 9000)])
def test_softmax(dev, shape):
    x = rng(10).standard_normal(shape).astype(np.float32)
    ref = orc.softmax(x, len(shape) - 1)
    dx = dev.from_numpy(x)
    assert_close(dev.softmax(dx, len(shape) - 1).to_numpy(), ref, 1e-6, "softmax")   # ops/softmax.rs:334
    dev.softmax(dx, len(shape) - 1, out=dx)   # in place, as the reference runs it
    assert_close(dx.to_numpy(), ref, 1e-6, "softmax in place")
    xh = x.astype(np.float16)
    assert_close(dev.softmax(dev.from_numpy(xh), len(shape) - 1).to_numpy(), orc.softmax(xh, len(shape) - 1), 1e-2, "softmax f16")   # the CPU path keeps its running sum in f16


def test_reduce(dev):
    from ratchet_b200 import capi
    x = rng(11).standard_normal((3, 40, 333)).astype(np.float32)
    dx = dev.from_numpy(x)
    assert_close(dev.reduce(capi.REDUCE_SUM, dx).to_numpy(), x.sum(-1), 1e-4)
    assert np.array_equal(dev.reduce(capi.REDUCE_MAX, dx).to_numpy(), x.max(-1))
    assert_close(dev.reduce(capi.REDUCE_MEAN, dx).to_numpy(), x.mean(-1), 1e-4)


@pytest.mark.parametrize("B,H,S,D,dim,off", [(1, 32, 1, 96, 96, 1024), (2, 3, 17, 64, 32, 5), (1, 4, 256, 128, 128, 0), (1, 1, 3, 80, 32, 4095)])
def test_rope(dev, B, H, S, D, dim, off):
    x = rng(12).standard_normal((B, H, S, D)).astype(np.float32)
    ref = orc.rope(x, dim, 10000.0, off)
    dx = dev.from_numpy(x)
    assert_close(dev.rope(dx, dim, 10000.0, off).to_numpy(), ref, 1e-4, "rope")
    dev.rope(dx, dim, 10000.0, off, out=dx)   # in place (ops/rope.rs supports_inplace)
    assert_close(dx.to_numpy(), ref, 1e-4, "rope in place")


# ------------------------------------------------------------------------------ indexing / copies: bit-exact
@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_reindex_ops(dev, dt):
    g = rng(13)
    x = g.standard_normal((2, 3, 20, 31)).astype(dt)
    dx = dev.from_numpy(x)
    for perm in ([0, 2, 1, 3], [3, 2, 1, 0], [0, 2, 3, 1], [1, 0, 3, 2], [0, 1, 3, 2], [0, 1, 2, 3]):
        assert np.array_equal(dev.permute(dx, perm).to_numpy(), orc.permute(x, perm)), perm
    x3 = g.standard_normal((1, 150, 38)).astype(dt)
    assert np.array_equal(dev.permute(dev.from_numpy(x3), [0, 2, 1]).to_numpy(), orc.permute(x3, [0, 2, 1]))
    x2 = g.standard_normal((37, 65)).astype(dt)
    assert np.array_equal(dev.permute(dev.from_numpy(x2), [1, 0]).to_numpy(), x2.T)
    for ranges in ([(0, 2), (1, 3), (4, 19), (7, 8)], [(0, 2), (0, 3), (0, 20), (8, 24)], [(1, 2), (0, 3), (0, 20), (0, 31)],
                   [(0, 2), (0, 3), (5, 6), (0, 31)], [(0, 2), (0, 3), (0, 20), (0, 31)]):
        assert np.array_equal(dev.slice(dx, ranges).to_numpy(), orc.slice_(x, ranges)), ranges
    for sshape, dshape in [((1, 3, 1, 31), (2, 3, 20, 31)), ((31,), (5, 31)), ((1,), (4, 9)), ((2, 1), (2, 64)), ((1, 1, 20, 1), (2, 3, 20, 31))]:
        s = g.standard_normal(sshape).astype(dt)
        assert np.array_equal(dev.broadcast(dev.from_numpy(s), dshape).to_numpy(), orc.broadcast(s, dshape)), (sshape, dshape)
    for dim, sizes in [(2, (3, 5, 1, 7, 2)), (0, (1, 2)), (3, (4, 4, 4, 4, 4, 4, 4, 4)), (1, (6,))]:
        shapes = []
        for n in sizes:
            s = [4, 2, 9, 16]
            s[dim] = n
            shapes.append(s)
        xs = [g.standard_normal(s).astype(dt) for s in shapes]
        assert np.array_equal(dev.concat([dev.from_numpy(a) for a in xs], dim).to_numpy(), orc.concat(xs, dim)), (dim, sizes)


def test_index_select(dev):
    from ratchet_b200 import RatchetCudaError, capi
    g = rng(14)
    table = g.standard_normal((512, 48)).astype(np.float32)
    ids = g.integers(0, 512, 64).astype(np.int32)
    dt_, di = dev.from_numpy(table), dev.from_numpy(ids)
    assert np.array_equal(dev.index_select(dt_, di, 0).to_numpy(), orc.index_select(table, ids, 0))
    ids1 = g.integers(0, 48, 7).astype(np.int32)
    assert np.array_equal(dev.index_select(dt_, dev.from_numpy(ids1), 1).to_numpy(), orc.index_select(table, ids1, 1))
    th = table.astype(np.float16)
    assert np.array_equal(dev.index_select(dev.from_numpy(th), di, 0).to_numpy(), orc.index_select(th, ids, 0))
    for half in (False, True):
        w = (g.standard_normal((320, 96)) * 0.02).astype(np.float16 if half else np.float32)
        buf = orc.quantize_q8(w)
        idq = g.integers(0, 320, 11).astype(np.int32)
        got = dev.index_select(dev.from_quantized(buf, capi.Q8_0H if half else capi.Q8_0F, (320, 96)), dev.from_numpy(idq), 0)
        assert got.dt == (capi.F16 if half else capi.F32)
        assert np.array_equal(bits(got.to_numpy()), bits(orc.index_select_q8(buf, (320, 96), half, idq, 0)))
    # an id outside the table is clamped and reported at the next synchronisation
    bad = dev.from_numpy(np.array([1, 9999], np.int32))
    out = dev.index_select(dt_, bad, 0)
    with pytest.raises(RatchetCudaError) as e:
        out.to_numpy()
    assert e.value.status == capi.ERR_BOUNDS
    assert np.array_equal(out.to_numpy()[1], table[511])   # flag cleared, data clamped


def test_cache_and_index_write(dev):
    from ratchet_b200 import capi
    g = rng(15)
    cache_h = np.zeros((1, 4, 64, 96), np.float16)
    dcache = dev.zeros(capi.F16, cache_h.shape)
    populated = 0
    for n in (5, 1, 1, 7):
        src = g.standard_normal((1, 4, n, 96)).astype(np.float16)
        ref = orc.cache(cache_h, src, 2, populated)
        got = dev.cache(dcache, dev.from_numpy(src), 2, populated)
        populated += n
        assert np.array_equal(got.to_numpy(), ref)
        assert np.array_equal(dcache.to_numpy(), cache_h)
    # append only (no materialised copy of the prefix)
    src = g.standard_normal((1, 4, 2, 96)).astype(np.float16)
    orc.cache(cache_h, src, 2, populated)
    assert dev.cache(dcache, dev.from_numpy(src), 2, populated, materialise=False) is None
    assert np.array_equal(dcache.to_numpy(), cache_h)
    dst = np.arange(2 * 3 * 8 * 10, dtype=np.float32).reshape(2, 3, 8, 10)
    blk = g.standard_normal((1, 2, 3, 4)).astype(np.float32)
    ddst = dev.from_numpy(dst)
    dev.index_write(ddst, dev.from_numpy(blk), [1, 0, 4, 5])
    assert np.array_equal(ddst.to_numpy(), orc.index_write(dst.copy(), blk, [1, 0, 4, 5]))
    d2 = dev.from_numpy(np.array([[1, 2, 3], [4, 5, 6]], np.float32))   # ops/index_write.rs:208-228
    dev.index_write(d2, dev.from_numpy(np.array([[7, 8]], np.float32)), [1, 1])
    assert np.array_equal(d2.to_numpy(), np.array([[1, 2, 3], [4, 7, 8]], np.float32))


@pytest.mark.parametrize("cin,lin,cout,stride", [(16, 64, 24, 1), (80, 3000, 384, 1), (384, 3000, 384, 2), (17, 129, 65, 2), (8, 3, 8, 1)])
def test_conv1d(dev, cin, lin, cout, stride):
    g = rng(16)
    x = g.standard_normal((1, cin, lin)).astype(np.float32)
    w = (g.standard_normal((cout, cin, 3)) * 0.05).astype(np.float32)
    b = g.standard_normal(cout).astype(np.float32)
    ref = orc.conv1d_k3(x, w, b, stride, 1)
    got = dev.conv1d(dev.from_numpy(x), dev.from_numpy(w), dev.from_numpy(b), stride, 1)
    assert got.shape == ref.shape
    assert_close(got.to_numpy(), ref, 1e-4, "conv1d")


@pytest.mark.parametrize("batch,cin,lin,cout,stride,pad", [(2, 36, 260, 40, 1, 1), (3, 68, 519, 100, 2, 1), (1, 32, 66, 32, 1, 0)])
def test_conv1d_unfolded_batches(dev, batch, cin, lin, cout, stride, pad):
    # shapes that take the unfold + tensor-core product: ragged channel tiles, several batches, no padding
    g = rng(17)
    x = g.standard_normal((batch, cin, lin)).astype(np.float32)
    w = (g.standard_normal((cout, cin, 3)) * 0.05).astype(np.float32)
    b = g.standard_normal(cout).astype(np.float32)
    ref = orc.conv1d_k3(x, w, b, stride, pad)
    got = dev.conv1d(dev.from_numpy(x), dev.from_numpy(w), dev.from_numpy(b), stride, pad)
    assert got.shape == ref.shape
    assert_close(got.to_numpy(), ref, 1e-4, "conv1d unfolded")
    nb = dev.conv1d(dev.from_numpy(x), dev.from_numpy(w), None, stride, pad)
    assert_close(nb.to_numpy(), orc.conv1d_k3(x, w, None, stride, pad), 1e-4, "conv1d unfolded, no bias")


def test_allocator_reuses_blocks(dev):
    from ratchet_b200 import capi
    a = dev.empty(capi.F32, (123457,))
    in_use0, reserved0 = dev.pool_stats()
    a.free()
    assert dev.pool_stats()[0] < in_use0
    b = dev.empty(capi.F32, (123457,))   # same size class: served from the pool, nothing new reserved
    in_use, reserved = dev.pool_stats()
    assert reserved == reserved0 and in_use == in_use0
    assert reserved >= in_use > 0
