"""The fused decode path (attention kernel and the CUDA-graph decode engine) against the CPU oracle
running the reference's own per-token graph (phi3/model.rs:134-156) on identical inputs."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc

from . import model_builders as mb
from .oracle_tensor import OTensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from ratchet_b200 import Device
    d = Device(0)
    yield d
    d.close()


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.abs(a - b).max() / (np.sqrt(np.mean(b * b)) + 1e-30)


def attention_reference(qkv, kc, vc, H, Hkv, hd, rope_dim, base, P):
    """float64 restatement of phi3/attn.rs:95-157 for one token with grouped KV heads; also appends."""
    q = qkv[: H * hd].reshape(H, hd).astype(np.float32)
    k = qkv[H * hd:(H + Hkv) * hd].reshape(Hkv, hd).astype(np.float32)
    v = qkv[(H + Hkv) * hd:].reshape(Hkv, hd)
    q = orc.rope(q.reshape(1, H, 1, hd), rope_dim, base, P).astype(np.float16).reshape(H, hd)
    k = orc.rope(k.reshape(1, Hkv, 1, hd), rope_dim, base, P).astype(np.float16).reshape(Hkv, hd)
    kc[:, P] = k
    vc[:, P] = v
    out = np.zeros((H, hd), np.float64)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    for h in range(H):
        kv = h // (H // Hkv)
        s = (q[h].astype(np.float32) @ kc[kv, : P + 1].astype(np.float32).T) * scale
        s = s.astype(np.float16).astype(np.float64)
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h] = p @ vc[kv, : P + 1].astype(np.float64)
    return out.reshape(-1)


@pytest.mark.parametrize("H,Hkv,hd,rope_dim,max_cache,P", [
    (32, 32, 96, 96, 4096, 1024), (32, 32, 96, 96, 4096, 0), (32, 32, 96, 96, 4096, 1), (4, 4, 96, 96, 64, 15), (4, 4, 96, 96, 64, 16),
    (4, 4, 96, 96, 64, 17), (8, 2, 64, 32, 512, 300), (8, 8, 128, 128, 1024, 1023), (32, 32, 96, 96, 4096, 4095)])
def test_attn_decode_kernel(dev, H, Hkv, hd, rope_dim, max_cache, P):
    from ratchet_b200 import capi
    g = np.random.Generator(np.random.PCG64(H * 1000 + P))
    qkv = g.standard_normal((H + 2 * Hkv) * hd).astype(np.float16)
    kc = np.zeros((Hkv, max_cache, hd), np.float16)
    vc = np.zeros((Hkv, max_cache, hd), np.float16)
    kc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
    vc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
    dq, dk, dv = dev.from_numpy(qkv), dev.from_numpy(kc), dev.from_numpy(vc)
    out = dev.empty(capi.F16, (H * hd,))
    for _ in range(2):   # the second call re-appends the same row and must give the same answer (counters reset)
        dev.check(dev._lib.rcu_attn_decode(dev.handle, dq.ptr, dk.ptr, dv.ptr, H, Hkv, hd, max_cache, rope_dim, 10000.0, P, out.ptr))
    ref = attention_reference(qkv, kc, vc, H, Hkv, hd, rope_dim, 10000.0, P)
    got = out.to_numpy().astype(np.float64)
    assert rel_err(got, ref) < 1e-2
    # KV append is a copy of the (rope'd) row: bit-exact
    k_dev = dk.to_numpy()
    assert np.array_equal(np.delete(k_dev, P, 1).view(np.uint16), np.delete(kc, P, 1).view(np.uint16))   # old rows untouched
    assert np.allclose(k_dev[:, P].astype(np.float32), kc[:, P].astype(np.float32), rtol=2e-3, atol=2e-3)   # rope'd row: f32 op + f16 rounding
    assert np.array_equal(dv.to_numpy().view(np.uint16), vc.view(np.uint16))


def test_allocating_entry_point_regrows_its_counters():
    """rcu_attn_decode keeps one scratch per device: a call with few heads and a long cache followed by one
    with more heads and a shorter cache (a smaller partial buffer, but more per-head counters) must not reuse
    the first call's counter array."""
    from ratchet_b200 import Device, capi
    dev = Device(0)
    try:
        for (H, Hkv, hd, rope_dim, max_cache, P) in [(8, 8, 128, 128, 8192, 2100), (32, 32, 64, 64, 2304, 2200)]:
            g = np.random.Generator(np.random.PCG64(H * 7 + P))
            qkv = g.standard_normal((H + 2 * Hkv) * hd).astype(np.float16)
            kc = np.zeros((Hkv, max_cache, hd), np.float16)
            vc = np.zeros((Hkv, max_cache, hd), np.float16)
            kc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
            vc[:, :P] = g.standard_normal((Hkv, P, hd)).astype(np.float16)
            dq, dk, dv = dev.from_numpy(qkv), dev.from_numpy(kc), dev.from_numpy(vc)
            out = dev.empty(capi.F16, (H * hd,))
            dev.check(dev._lib.rcu_attn_decode(dev.handle, dq.ptr, dk.ptr, dv.ptr, H, Hkv, hd, max_cache, rope_dim, 10000.0, P, out.ptr))
            got = out.to_numpy().astype(np.float32)
            cpu = attention_reference(qkv, kc, vc, H, Hkv, hd, rope_dim, 10000.0, P)
            assert rel_err(got, cpu) < 1e-2, f"H={H} P={P}"
    finally:
        dev.close()


def test_decoder_matches_reference_graph(dev):
    """Two layers of Phi-3-mini (full widths, vocab 32064, 1024 prior KV positions, Q8_0H weights with
    f16 activations as the reference loads them on an f16-capable device), three greedy steps: the
    fused engine must agree with the oracle running the reference's per-token graph."""
    W = mb.phi3_weights(3, n_layers=2, quant="q8h")
    act = np.float16
    ref_model = mb.phi3_model(OTensor, None, W, 1024, act)
    dec = mb.phi3_decoder(dev, W, 1024)
    assert dec.position == 1024
    tok = 777
    for step in range(3):
        ref = ref_model.schedule(OTensor.from_data(np.array([[tok]], np.int32))).full().to_numpy().reshape(-1)
        ref_model.kv_cache.update(1)
        got = dec.step(tok).astype(np.float32).reshape(-1)
        e = rel_err(got, ref)
        assert e < 1e-2, f"step {step}: logits differ, normalised max error {e:.3e}"
        assert int(got.argmax()) == int(ref.argmax())
        assert dec.position == 1025 + step
        tok = int(ref.argmax())
    # all layers as one persistent kernel (rope table, embedding gather, layers, lm_head, arg-max), or five kernels per layer
    assert dec.kernels_per_step in (5, 2 + 5 * 2 + 2)
    # caches hold the same appended rows
    for li in range(2):
        k_ref = ref_model.kv_cache[li].k_cache.to_numpy()[0, :, 1024:1027].astype(np.float32)
        k_dev = dec._keep[0][li].k_cache.to_numpy()[:, 1024:1027].astype(np.float32)
        assert rel_err(k_dev, k_ref) < 1e-2


def test_decoder_across_the_attention_kernel_switch(dev):
    """The attention kernel changes with the cached length (one cluster per head up to 2048 positions,
    one CTA per 64-position tile beyond): a narrow one-layer model stepping from 2046 to 2050 cached
    positions, from a stream of its own so that the steps replay (and re-capture) a CUDA graph."""
    import torch
    from ratchet_b200 import Device
    stream = torch.cuda.Stream()
    sdev = Device(0, stream=stream.cuda_stream)
    try:
        W = mb.phi3_weights(9, n_layers=1, d=512, n_heads=8, ffn=1024, vocab=4096, quant="q8h")
        ref_model = mb.phi3_model(OTensor, None, W, 2046, np.float16)
        dec = mb.phi3_decoder(sdev, W, 2046)
        tok = 5
        for step in range(5):
            ref = ref_model.schedule(OTensor.from_data(np.array([[tok]], np.int32))).full().to_numpy().reshape(-1)
            ref_model.kv_cache.update(1)
            got = dec.step(tok).astype(np.float32).reshape(-1)
            assert rel_err(got, ref) < 1e-2, f"step {step} (position {2046 + step})"
            assert int(got.argmax()) == int(ref.argmax())
            tok = int(ref.argmax())
        assert dec.position == 2051
        dec.close()
    finally:
        sdev.close()


def test_decoder_greedy_loop_on_device(dev):
    """Greedy generation without a host round trip: the arg-max id feeds the next step on the device;
    the result equals stepping from the host with the logits' arg-max."""
    W = mb.phi3_weights(4, n_layers=1, d=512, n_heads=8, ffn=1024, vocab=4096, quant="q8h")
    a = mb.phi3_decoder(dev, W, 5, max_cache=64)
    b = mb.phi3_decoder(dev, W, 5, max_cache=64)
    tok = 11
    host_tokens = []
    for _ in range(6):
        logits = a.step(tok)
        tok = int(logits.reshape(-1).argmax())
        host_tokens.append(tok)
    dev.h2d(b.next_token.ptr, np.array([11], np.int32))
    dev_tokens = []
    for _ in range(6):
        b.step_device(token_ptr=b.next_token.ptr, argmax=True)
        dev_tokens.append(int(b.next_token.to_numpy()[0]))
    assert dev_tokens == host_tokens
    assert a.position == b.position == 11


def test_decoder_kernel_per_phase_fallback(dev):
    """A model whose rows are not whole 256-element runs (d_model 480 = 5 heads of 96) cannot use the rings of
    the data-flow kernel: the decoder keeps the kernel-per-phase step (five kernels per layer), with the same
    results against the oracle's graph."""
    W = mb.phi3_weights(21, n_layers=2, d=480, n_heads=5, ffn=1024, vocab=2048, quant="q8h")
    ref_model = mb.phi3_model(OTensor, None, W, 70, np.float16, max_cache=128)
    dec = mb.phi3_decoder(dev, W, 70, max_cache=128)
    tok = 3
    for step in range(3):
        ref = ref_model.schedule(OTensor.from_data(np.array([[tok]], np.int32))).full().to_numpy().reshape(-1)
        ref_model.kv_cache.update(1)
        got = dec.step(tok).astype(np.float32).reshape(-1)
        assert rel_err(got, ref) < 1e-2, f"step {step}"
        tok = int(ref.argmax())
    assert dec.kernels_per_step == 2 + 5 * 2 + 2
    with pytest.raises(Exception):
        dec.profile_step()              # per-job time stamps exist only for the data-flow kernel


def test_decoder_profile_step_reports_every_job(dev):
    W = mb.phi3_weights(4, n_layers=2, d=512, n_heads=8, ffn=1024, vocab=4096, quant="q8h")
    dec = mb.phi3_decoder(dev, W, 5, max_cache=64)
    assert dec.kernels_per_step in (0, 5)
    dev.h2d(dec.token.ptr, np.array([11], np.int32))
    stamps = dec.profile_step()
    n_jobs = 5 * 2 + 1
    assert stamps.size == 2 * n_jobs + 1 + 24
    t = stamps[: 2 * n_jobs + 1].astype(np.int64)
    assert (np.diff(t) >= 0).all() and t[-1] > t[0]          # one clock, in job order
    assert dec.position == 6
