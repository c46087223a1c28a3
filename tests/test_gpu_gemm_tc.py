"""The tcgen05 prefill GEMM (Linear convention, f16 activations) against the CPU oracle:
dequantise (bit-exact) then f32-accumulated matmul, within 1e-2 of the result's scale."""
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


def check(got, ref, tol, what):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, what
    scale = np.sqrt(np.mean(ref * ref)) + 1e-30
    bad = np.abs(got - ref) > tol * (scale + np.abs(ref))
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside {tol}; max abs {np.abs(got - ref).max():.3e}, rms {scale:.3e}"


# (M, N, K): full tiles, ragged M / N / K edges, several k-steps beyond the pipeline depth, both tile widths
SHAPES = [(128, 256, 256), (512, 512, 1024), (100, 200, 136), (37, 64, 64), (2048, 256, 512), (130, 1032, 3072), (1500, 384, 384),
          # the CTA-pair kernel (at least 37 tiles of 256 x 256): full tiles; ragged M, N and K; more tiles than CTA pairs
          # (persistent loop, both accumulator buffers, the stage ring wrapping across tiles); one k-step only
          (1024, 2560, 320), (1000, 2504, 328), (2048, 4096, 512), (1300, 5000, 136), (2048, 8192, 64),
          # 88 tiles on 74 pairs (a short last round) with a ragged last N tile
          (1024, 5600, 320),
          # few tiles and a long K: K is cut into slices (the last one a single k-step) that a second kernel sums
          (128, 512, 1088), (300, 640, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_tc_f16(dev, M, N, K, with_bias):
    g = np.random.Generator(np.random.PCG64(M * 7 + N + K))
    w = (g.standard_normal((N, K)) * 0.05).astype(np.float16)
    x = g.standard_normal((M, K)).astype(np.float16)
    b = g.standard_normal(N).astype(np.float16) if with_bias else None
    ref = orc.matmul(w, x, b, False, True, True)
    y = dev.matmul(dev.from_numpy(w), dev.from_numpy(x), None if b is None else dev.from_numpy(b), False, True, True)
    assert y.shape == (M, N)
    check(y.to_numpy(), ref, 1e-2, f"f16 {M}x{N}x{K}")


# batched f16 products A[b, M, K] . B[b, K, N] (or B as [b, N, K] with trans_rhs): Whisper-tiny's q.k^T and weights.v over six
# heads of 1500 positions (K = 1500 is not a multiple of 8: padded scratch rows; N = 1500 is not one either: 8-byte stores),
# a shape with whole tiles, and one with ragged M
@pytest.mark.parametrize("b,M,K,N,trans_rhs", [(6, 1500, 64, 1500, False), (6, 1500, 1500, 64, False), (2, 256, 128, 256, True),
                                                (3, 200, 72, 132, False), (2, 384, 1000, 64, True)])
def test_gemm_tc_batched_f16(dev, b, M, K, N, trans_rhs):
    g = np.random.Generator(np.random.PCG64(b * M + K + N))
    a = (g.standard_normal((1, b, M, K)) * 0.5).astype(np.float16)
    bm = (g.standard_normal((1, b, N, K) if trans_rhs else (1, b, K, N)) * 0.5).astype(np.float16)
    ref = orc.matmul(a, bm, None, False, trans_rhs, False)
    y = dev.matmul(dev.from_numpy(a), dev.from_numpy(bm), None, False, trans_rhs, False)
    assert y.shape == (1, b, M, N)
    check(y.to_numpy(), ref, 1e-2, f"batched f16 {b}x{M}x{K}x{N}")


@pytest.mark.parametrize("kind", ["Q8_0H", "Q4_KH"])
@pytest.mark.parametrize("M,N,K", [(128, 512, 768), (512, 256, 3072), (77, 96, 512), (64, 512, 2048), (48, 1024, 4096)])
def test_gemm_tc_quantised(dev, kind, M, N, K):
    from ratchet_b200 import capi
    g = np.random.Generator(np.random.PCG64(M + N + K))
    w = (g.standard_normal((N, K)) * 0.02)
    x = g.standard_normal((2, M, K)).astype(np.float16)     # a leading batch dimension folds into M
    if kind == "Q8_0H":
        buf = orc.quantize_q8(w.astype(np.float16))
        wd = orc.dequantize_q8(buf, (N, K), True)
        dt = capi.Q8_0H
    else:
        buf = orc.quantize_q4k(w.astype(np.float32), True)
        wd = orc.dequantize_q4k(buf, (N, K), True)
        dt = capi.Q4_KH
    ref = orc.matmul(wd, x, None, False, True, True)
    y = dev.matmul(dev.from_quantized(buf, dt, (N, K)), dev.from_numpy(x), None, False, True, True)
    assert y.shape == (2, M, N)
    check(y.to_numpy(), ref, 1e-2, f"{kind} {M}x{N}x{K}")


@pytest.fixture(scope="module")
def config3_weight():
    """W [8192, 3072] N(0, 0.02) in ratchet Q4_K with f16 super-block scales, and its dequantised form."""
    g = np.random.Generator(np.random.PCG64(0))
    N, K = 8192, 3072
    w = (g.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
    buf = orc.quantize_q4k(w, True)
    assert buf.size == 14155776          # 144 bytes per 256-weight super-block
    return buf, orc.dequantize_q4k(buf, (N, K), True)


@pytest.mark.parametrize("M", [128, 256, 512, 2048])
def test_config3_q4k_prefill_shape(dev, config3_weight, M):
    """Config 3 at its three sizes (and 256, the last size of the fused kernel): x [M, 3072] f16 N(0,1),
    W [8192, 3072] in ratchet Q4_K, out [M, 8192] f16.  M <= 256 runs the kernel that converts Q4_K tiles in
    shared memory; M = 512 and 2048 convert the matrix once into scratch and run the CTA-pair f16 kernel:
    all against dequantise -> matmul."""
    from ratchet_b200 import capi
    N, K = 8192, 3072
    buf, wd = config3_weight
    x = np.random.Generator(np.random.PCG64(M)).standard_normal((M, K)).astype(np.float16)
    ref = orc.matmul(wd, x, None, False, True, True)
    y = dev.matmul(dev.from_quantized(buf, capi.Q4_KH, (N, K)), dev.from_numpy(x), None, False, True, True)
    assert y.shape == (M, N)
    check(y.to_numpy(), ref, 1e-2, f"config 3, M={M}")


# f32 Linear on the tensor cores (split TF32): the f32 bar, 1e-4 of the result's scale
F32_SHAPES = [(64, 10240, 2560), (128, 256, 256), (100, 200, 136), (37, 64, 36), (1500, 384, 384), (1500, 1536, 384), (300, 2560, 10240),
              # grids that fill under half of the SMs with a long K: K is split over CTAs and the slices summed in order
              (64, 2560, 10240), (100, 192, 2000), (1500, 384, 1536),
              # grids of one and two rounds of CTAs with either tile width
              (300, 4800, 256), (200, 6912, 128)]


@pytest.mark.parametrize("M,N,K", F32_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_tc_f32(dev, M, N, K, with_bias):
    g = np.random.Generator(np.random.PCG64(M * 3 + N + K))
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = g.standard_normal((M, K)).astype(np.float32)
    b = g.standard_normal(N).astype(np.float32) if with_bias else None
    ref = orc.matmul(w, x, b, False, True, True)
    y = dev.matmul(dev.from_numpy(w), dev.from_numpy(x), None if b is None else dev.from_numpy(b), False, True, True)
    assert y.shape == (M, N)
    check(y.to_numpy(), ref, 1e-4, f"f32 {M}x{N}x{K}")


# batched f32 products of the attention kind (whisper/mha.rs:82-86): A[b,M,K] . B[b,K,N], and B given transposed
@pytest.mark.parametrize("b,M,K,N,tr", [(6, 1500, 64, 1500, False), (6, 1500, 1500, 64, False), (3, 100, 36, 72, False),
                                        (2, 130, 64, 200, True), (1, 64, 128, 64, False)])
def test_gemm_tc_f32_batched(dev, b, M, K, N, tr):
    g = np.random.Generator(np.random.PCG64(b * 1000 + M + K + N))
    a = g.standard_normal((b, M, K)).astype(np.float32)
    w = (g.standard_normal((b, N, K) if tr else (b, K, N)) * 0.1).astype(np.float32)
    ref = orc.matmul(a, w, None, False, tr, False)
    y = dev.matmul(dev.from_numpy(a), dev.from_numpy(w), None, False, tr, False)
    assert y.shape == (b, M, N)
    check(y.to_numpy(), ref, 1e-4, f"batched f32 {b}x{M}x{K}x{N} tr={tr}")
