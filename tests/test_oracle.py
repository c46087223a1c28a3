"""The CPU oracle against torch, using the ground truths and tolerances of the reference's own
per-op tests (crates/ratchet-core/src/ops/*.rs `mod tests`), plus bit-level checks of the parts
quant.rs defines exactly."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc


def rng(seed=0):
    return np.random.Generator(np.random.PCG64(seed))


def close(a, b, atol, rtol):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.all(np.abs(a - b) <= atol + rtol * np.abs(b))  # tensor.rs:1039-1043


# ---------------------------------------------------------------- quantisation (bit-defined)
@pytest.mark.parametrize("half", [False, True])
def test_q8_layout_and_bits(half):
    x = rng(1).standard_normal((64, 96)).astype(np.float16 if half else np.float32)
    buf = orc.quantize_q8(x)
    n = x.size
    # dtype/blocks.rs:69-82: qs padded to 256, then scales padded to 256
    assert buf.size == (n + 255) // 256 * 256 + ((n // 32) * (2 if half else 4) + 255) // 256 * 256
    qs = buf[:n].view(np.int8).reshape(-1, 32)
    d = buf[orc.q8_scale_offset(n):][: (n // 32) * (2 if half else 4)].view(np.float16 if half else np.float32)
    xb = x.reshape(-1, 32)
    T = np.float16 if half else np.float32
    d_ref = (np.abs(xb).max(1).astype(T) / T(127)).astype(T)  # quant.rs:31-36
    assert np.array_equal(d, d_ref)
    v = (xb / d_ref[:, None]).astype(T).astype(np.float64)
    q_ref = np.where(v >= 0, np.floor(v + 0.5), np.ceil(v - 0.5)).astype(np.int8)  # round half away
    assert np.array_equal(qs, q_ref)
    # never emits -128
    assert qs.min() >= -127
    # dequantise: quant.rs:118-127, product rounded once in FP
    dq = orc.dequantize_q8(buf, x.shape, half)
    dq_ref = (qs.astype(T) * d_ref[:, None]).astype(T).reshape(x.shape)
    assert np.array_equal(dq.view(np.uint16 if half else np.uint32), dq_ref.view(np.uint16 if half else np.uint32))


def test_q8_zero_block_and_minus128():
    x = np.zeros(64, np.float32)
    x[32:] = rng(2).standard_normal(32)
    buf = orc.quantize_q8(x)
    assert np.all(buf[:32] == 0)  # 0/0 = NaN -> 0 (Rust `as i32`)
    # a GGUF file may carry -128; CPU dequantisation keeps it (quant.rs:121-127)
    buf[0] = 0x80
    buf[orc.q8_scale_offset(64):][:4] = np.array([0.5], np.float32).view(np.uint8)
    assert orc.dequantize_q8(buf, (64,), False)[0] == -64.0


@pytest.mark.parametrize("half", [False, True])
def test_quantisation_reflexivity(half):
    # quant.rs:171-190: 64x64 randn, atol=rtol 0.1 (Q8) / 0.3 (4-bit absmax)
    x = rng(3).standard_normal((64, 64)).astype(np.float16 if half else np.float32)
    assert close(orc.dequantize_q8(orc.quantize_q8(x), x.shape, half), x, 0.1, 0.1)
    assert close(orc.dequantize_q4abs(orc.quantize_q4abs(x), x.shape, half), x, 0.3, 0.3)


@pytest.mark.parametrize("half", [False, True])
def test_q4k_layout_and_decode(half):
    x = (rng(4).standard_normal((8, 512)) * 0.02).astype(np.float32)
    buf = orc.quantize_q4k(x, half)
    n = x.size
    nb = n // 256
    fp = 2 if half else 4
    a = lambda v: (v + 255) // 256 * 256
    off = orc.q4k_offsets(n, half)
    # dtype/blocks.rs:124-148
    assert off == [0, a(n // 2), a(n // 2) + a(nb * 12), a(n // 2) + a(nb * 12) + a(nb * fp)]
    assert buf.size == off[3] + a(nb * fp)
    dq = orc.dequantize_q4k(buf, x.shape, half).astype(np.float32)
    # independent numpy decode following ops/matmul/quantized.rs:158-266
    T = np.float16 if half else np.float32
    qs = buf[off[0]:off[0] + n // 2].reshape(nb, 4, 32)
    sc = buf[off[1]:off[1] + nb * 12].reshape(nb, 12).astype(np.uint32)
    dmin = buf[off[2]:off[2] + nb * fp].view(T)
    d = buf[off[3]:off[3] + nb * fp].view(T)
    ref = np.zeros((nb, 8, 32), np.float64)
    for j in range(8):
        if j < 4:
            s = sc[:, j] & 63
            m = sc[:, j + 4] & 63
        else:
            s = (sc[:, j + 4] & 0xF) | ((sc[:, j - 4] >> 6) << 4)
            m = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
        delta = (s.astype(T) * d).astype(T)
        mn = (m.astype(T) * dmin).astype(T)
        q = (qs[:, j // 2, :] >> 4) if (j & 1) else (qs[:, j // 2, :] & 0xF)
        ref[:, j, :] = (q.astype(np.float64) * delta[:, None].astype(np.float64) - mn[:, None].astype(np.float64))
    ref = ref.astype(T).astype(np.float32).reshape(x.shape)  # fma: one rounding
    assert np.array_equal(dq, ref)
    # the quantiser itself is this repository's own; it only has to be a sane 4-bit code
    assert np.abs(dq - x).max() < 0.02 * 6 / 15


# ---------------------------------------------------------------- matmul
CASES = [(False, False, False), (True, False, False), (False, True, False), (False, False, True),
         (True, True, False), (False, True, True)]


@pytest.mark.parametrize("tl,tr,td", CASES)
def test_sgemm_vs_torch(tl, tr, td):
    # ops/matmul/mod.rs:818-946: B 1..3, M,K,N 1..256, atol=rtol=1e-4
    g = rng(5)
    for _ in range(4):
        B, M, K, N = g.integers(1, 4), g.integers(1, 257), g.integers(1, 257), g.integers(1, 257)
        a = g.standard_normal((B, K, M) if tl else (B, M, K)).astype(np.float32)
        b = g.standard_normal((B, N, K) if tr else (B, K, N)).astype(np.float32)
        ta, tb = torch.from_numpy(a), torch.from_numpy(b)
        ref = (ta.transpose(-1, -2) if tl else ta) @ (tb.transpose(-1, -2) if tr else tb)
        if td:
            ref = ref.transpose(-1, -2)
        out = orc.matmul(a, b, None, tl, tr, td)
        assert out.shape == tuple(ref.shape)
        assert close(out, ref.numpy(), 1e-4, 1e-4)


def test_linear_convention_with_bias_and_stack_broadcast():
    # ratchet-nn/src/linear.rs:17-24: w.gemm(x, bias, false, true, true) == x @ w.T + b
    g = rng(6)
    w = g.standard_normal((48, 32)).astype(np.float32)
    x = g.standard_normal((2, 5, 32)).astype(np.float32)
    b = g.standard_normal(48).astype(np.float32)
    out = orc.matmul(w, x, b, False, True, True)
    assert out.shape == (2, 5, 48)
    assert close(out, x @ w.T + b, 1e-4, 1e-4)
    xh, wh, bh = x.astype(np.float16), w.astype(np.float16), b.astype(np.float16)
    outh = orc.matmul(wh, xh, bh, False, True, True)
    assert outh.dtype == np.float16
    assert close(outh, xh.astype(np.float32) @ wh.astype(np.float32).T + bh.astype(np.float32), 2e-2, 1e-2)


def test_gemv_q8_matches_dequant_matmul():
    g = rng(7)
    for half in (False, True):
        T = np.float16 if half else np.float32
        w = (g.standard_normal((40, 96)) * 0.02).astype(T)
        x = g.standard_normal(96).astype(T)
        buf = orc.quantize_q8(w)
        wd = orc.dequantize_q8(buf, w.shape, half)
        ref = orc.matmul(wd, x.reshape(1, 96), None, False, True, True).reshape(-1)
        y = orc.gemv_q8(buf, 40, 96, half, x)
        assert close(y, ref, 1e-5 if not half else 2e-3, 1e-5 if not half else 2e-3)


# ---------------------------------------------------------------- elementwise
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary_vs_torch(op):
    g = rng(8)
    a = g.standard_normal((2, 33, 17)).astype(np.float32)
    b = g.standard_normal((2, 33, 17)).astype(np.float32)
    ref = getattr(torch, op)(torch.from_numpy(a), torch.from_numpy(b)).numpy()
    assert close(orc.binary(op, a, b), ref, 1e-4, 1e-4)  # ops/binary.rs:319
    ah, bh = a.astype(np.float16), b.astype(np.float16)
    refh = getattr(torch, op)(torch.from_numpy(ah), torch.from_numpy(bh)).numpy()
    assert np.array_equal(orc.binary(op, ah, bh).view(np.uint16), refh.view(np.uint16))


@pytest.mark.parametrize("op", list(orc.UNARY_OPS))
def test_unary_vs_torch(op):
    g = rng(9)
    x = g.standard_normal((2, 128, 65)).astype(np.float32)
    if op in ("log", "sqrt"):
        x = np.abs(x) + 1e-3
    t = torch.from_numpy(x)
    if op == "gelu":
        ref = torch.nn.functional.gelu(t, approximate="tanh")
    elif op == "silu":
        ref = torch.nn.functional.silu(t)
    elif op == "relu":
        ref = torch.relu(t)
    else:
        ref = getattr(torch, op)(t)
    tol = 5e-2 if op in ("gelu", "tanh") else 1e-4  # ops/unary.rs:440-443
    assert close(orc.unary(op, x), ref.numpy(), tol, tol)
    # f16: every operation rounds (half crate semantics) -> loose check only
    xh = x.astype(np.float16)
    th = torch.from_numpy(xh.astype(np.float32))
    refh = {"gelu": lambda v: torch.nn.functional.gelu(v, approximate="tanh"), "silu": torch.nn.functional.silu,
            "relu": torch.relu}.get(op, getattr(torch, op, None))(th)
    assert close(orc.unary(op, xh), refh.numpy(), 2e-2, 2e-2)


def test_cast():
    x = rng(10).standard_normal(1000).astype(np.float32)
    h = orc.cast(x, orc.F32, orc.F16)
    assert np.array_equal(h.view(np.uint16), x.astype(np.float16).view(np.uint16))
    assert np.array_equal(orc.cast(h, orc.F16, orc.F32), h.astype(np.float32))
    b = orc.cast(x, orc.F32, orc.BF16)
    assert np.array_equal(b, torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    # cpu/mod.rs:116-125: f32 <-> i32/u32 are bit reinterpretations
    assert np.array_equal(orc.cast(x, orc.F32, orc.I32), x.view(np.int32))
    assert np.array_equal(orc.cast(x.view(np.uint32), orc.U32, orc.F32), x)


# ---------------------------------------------------------------- norm / softmax / rope
def test_norms_vs_torch():
    g = rng(11)
    for _ in range(4):
        B, M, N = g.integers(1, 4), g.integers(1, 257), g.integers(1, 257)
        x = g.standard_normal((B, M, N)).astype(np.float32)
        s = g.standard_normal(N).astype(np.float32)
        b = g.standard_normal(N).astype(np.float32)
        ref = torch.nn.functional.layer_norm(torch.from_numpy(x), (N,), torch.from_numpy(s), torch.from_numpy(b), 1e-5)
        assert close(orc.layer_norm(x, s, b, 1e-5), ref.numpy(), 1e-4, 1e-4)  # ops/norm/mod.rs:467
        ref = torch.nn.functional.layer_norm(torch.from_numpy(x), (N,), torch.from_numpy(s), None, 1e-5)
        assert close(orc.layer_norm(x, s, None, 1e-5), ref.numpy(), 1e-4, 1e-4)
        t = torch.from_numpy(x)
        ref = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5) * torch.from_numpy(s)
        assert close(orc.rms_norm(x, s, 1e-5), ref.numpy(), 1e-4, 1e-4)


def test_softmax_vs_torch():
    g = rng(12)
    x = g.standard_normal((2, 77, 130)).astype(np.float32)
    ref = torch.softmax(torch.from_numpy(x), -1).numpy()
    assert close(orc.softmax(x, 2), ref, 1e-6, 1e-6)  # ops/softmax.rs:334


def test_rope_vs_float64():
    # ops/rope.rs:269-312 checks against MLX nn.RoPE(traditional=False) at 1e-2
    g = rng(13)
    B, H, S, D, dim, off, base = 2, 3, 17, 64, 32, 5, 10000.0
    x = g.standard_normal((B, H, S, D)).astype(np.float32)
    half = dim // 2
    inv = base ** (-np.arange(half) / half)
    th = (np.arange(S) + off)[:, None] * inv[None, :]
    x1, x2 = x[..., :half].astype(np.float64), x[..., half:dim].astype(np.float64)
    ref = np.concatenate([x1 * np.cos(th) - x2 * np.sin(th), x1 * np.sin(th) + x2 * np.cos(th), x[..., dim:]], -1)
    assert close(orc.rope(x, dim, base, off), ref, 1e-4, 1e-4)


# ---------------------------------------------------------------- indexing / copies (exact)
def test_concat_permute_slice_broadcast_select():
    g = rng(14)
    xs = [g.standard_normal((4, 2, n, 16)).astype(np.float32) for n in (3, 5, 1, 7, 2)]
    assert np.array_equal(orc.concat(xs, 2), np.concatenate(xs, 2))
    x = g.standard_normal((2, 3, 20, 31)).astype(np.float32)
    for perm in ([0, 2, 1, 3], [3, 2, 1, 0], [0, 2, 3, 1], [1, 0, 3, 2]):
        assert np.array_equal(orc.permute(x, perm), np.transpose(x, perm))
    assert np.array_equal(orc.permute(x[0, 0], [1, 0]), x[0, 0].T)
    assert np.array_equal(orc.slice_(x, [(0, 2), (1, 3), (4, 19), (7, 8)]), x[0:2, 1:3, 4:19, 7:8])
    s = g.standard_normal((1, 3, 1, 31)).astype(np.float16)
    assert np.array_equal(orc.broadcast(s, (2, 3, 20, 31)), np.broadcast_to(s, (2, 3, 20, 31)))
    v = g.standard_normal(31).astype(np.float32)
    assert np.array_equal(orc.broadcast(v, (5, 31)), np.broadcast_to(v, (5, 31)))
    # the reference's vector fast path (cpu/reindex.rs:165-173) repeats each element
    v5 = g.standard_normal(5).astype(np.float32)
    assert np.array_equal(orc.broadcast(v5, (5, 4), vector_fast_path=True), np.repeat(v5, 4).reshape(5, 4))
    table = g.standard_normal((50, 16)).astype(np.float32)
    ids = g.integers(0, 50, 9).astype(np.int32)
    assert np.array_equal(orc.index_select(table, ids, 0), table[ids])
    ids1 = g.integers(0, 16, 4).astype(np.int32)
    assert np.array_equal(orc.index_select(table, ids1, 1), table[:, ids1])
    wq = orc.quantize_q8(table.reshape(25, 32))
    full = orc.dequantize_q8(wq, (25, 32), False)
    idq = g.integers(0, 25, 6).astype(np.int32)
    assert np.array_equal(orc.index_select_q8(wq, (25, 32), False, idq, 0), full[idq])


def test_cache_and_index_write():
    g = rng(15)
    cache = np.zeros((1, 2, 16, 8), np.float32)
    populated = 0
    chunks = []
    for n in (3, 1, 4):
        src = g.standard_normal((1, 2, n, 8)).astype(np.float32)
        chunks.append(src)
        out = orc.cache(cache, src, 2, populated)
        populated += n
        assert np.array_equal(out, np.concatenate(chunks, 2))  # ops/cache.rs:267-302
        assert np.array_equal(cache[:, :, :populated], out)
    # ops/index_write.rs:208-228
    dst = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    orc.index_write(dst, np.array([[7, 8]], np.float32), [1, 1])
    assert np.array_equal(dst, np.array([[1, 2, 3], [4, 7, 8]], np.float32))


def test_conv1d_vs_torch():
    g = rng(16)
    for (cin, lin, cout, stride) in [(16, 64, 24, 1), (80, 300, 48, 1), (48, 301, 48, 2)]:
        x = g.standard_normal((1, cin, lin)).astype(np.float32)
        w = g.standard_normal((cout, cin, 3)).astype(np.float32)
        b = g.standard_normal(cout).astype(np.float32)
        ref = torch.nn.functional.conv1d(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b), stride=stride, padding=1)
        out = orc.conv1d_k3(x, w, b, stride, 1)
        assert out.shape == tuple(ref.shape)
        assert close(out, ref.numpy(), 5e-3, 5e-3)  # ops/conv.rs:342
