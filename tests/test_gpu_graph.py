"""The lazy Tensor graph on the CUDA device: resolver semantics (execution order, in-place rule,
buffer planning, views) and the benchmark configurations scheduled through the same caller code on
the CUDA device and on the CPU oracle."""
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


# ------------------------------------------------------------------------------ resolver semantics
def test_lazy_chain_inplace_and_stats(dev):
    from ratchet_b200 import Tensor, last_resolve_stats
    g = np.random.Generator(np.random.PCG64(0))
    a = g.standard_normal((4, 33, 65)).astype(np.float32)
    b = g.standard_normal((4, 33, 65)).astype(np.float32)
    ta, tb = Tensor.from_data(a, device=dev), Tensor.from_data(b, device=dev)
    assert ta.resolved() and ta.strong_count() == 1
    y = ta.add(tb)            # ta and tb stay referenced by this scope -> cannot be overwritten
    assert not y.resolved() and ta.strong_count() == 2
    z = y.gelu().mul(tb).exp()
    del y                      # drop the handle: the chain owns it alone now
    z.resolve()
    st = last_resolve_stats(dev)
    assert st["launched"] == 4
    assert st["inplace"] == 3          # gelu, mul, exp run in place on the add's buffer (tensor.rs:823-824)
    assert st["buffers"] == 1
    ref = orc.unary("exp", orc.binary("mul", orc.unary("gelu", orc.binary("add", a, b)), b))
    assert np.allclose(z.to_numpy(), ref, rtol=1e-4, atol=1e-4)
    assert np.array_equal(ta.to_numpy(), a) and np.array_equal(tb.to_numpy(), b)   # constants untouched


def test_held_intermediate_is_not_overwritten(dev):
    from ratchet_b200 import Tensor, last_resolve_stats
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    ta = Tensor.from_data(a, device=dev)
    mid = ta.neg()
    out = mid.abs().sqrt()
    out.resolve()                      # `mid` is still held: abs must not run in place on it
    assert last_resolve_stats(dev)["inplace"] == 1
    assert np.array_equal(mid.to_numpy(), -a)
    assert np.allclose(out.to_numpy(), np.sqrt(a))


def test_inplace_on_owned_constant(dev):
    from ratchet_b200 import Tensor, last_resolve_stats
    a = np.linspace(-3, 3, 64, dtype=np.float32).reshape(8, 8)
    t = Tensor.from_data(a, device=dev)
    ptr = t.data_ptr()
    r = t.relu()
    del t                              # the op is now the constant's sole owner
    r.resolve()
    assert last_resolve_stats(dev)["inplace"] == 1 and r.data_ptr() == ptr
    assert np.array_equal(r.to_numpy(), np.maximum(a, 0))


def test_views_share_storage_and_extend_liveness(dev):
    from ratchet_b200 import Tensor
    a = np.random.Generator(np.random.PCG64(1)).standard_normal((6, 8)).astype(np.float32)
    t = Tensor.from_data(a, device=dev)
    v = t.view([2, 3, 8])
    assert v.resolved() and v.data_ptr() == t.data_ptr()      # tensor.rs:454-461
    s = t.sin()                        # unresolved source
    v2 = s.view([48])
    assert not v2.resolved()
    w = v2.view([4, 12]).permute([1, 0])
    out = w.add(Tensor.from_data(np.ones((12, 4), np.float32), device=dev))
    assert np.allclose(out.to_numpy(), np.sin(a).reshape(4, 12).T + 1, atol=1e-6)
    assert v2.resolved() and v2.data_ptr() == s.data_ptr()
    with pytest.raises(Exception):
        t.view([5, 5])


def test_cast_to_same_dtype_is_identity(dev):
    from ratchet_b200 import Tensor, capi
    t = Tensor.from_data(np.zeros((2, 2), np.float32), device=dev)
    same = t.full()
    assert same.data_ptr() == t.data_ptr() and t.strong_count() == 2   # tensor.rs:315-318
    assert t.half().dt() == capi.F16


def test_binary_broadcast_both_sides(dev):
    from ratchet_b200 import Tensor
    g = np.random.Generator(np.random.PCG64(2))
    a = g.standard_normal((1, 6, 1, 9)).astype(np.float32)
    b = g.standard_normal((5, 1)).astype(np.float32)
    out = Tensor.from_data(a, device=dev).mul(Tensor.from_data(b, device=dev))
    assert out.shape() == (1, 6, 5, 9)
    assert np.array_equal(out.to_numpy(), a * b)
    with pytest.raises(Exception):
        Tensor.from_data(a, device=dev).add(Tensor.from_data(np.zeros((4, 2), np.float32), device=dev))   # BroadcastingFailed


def test_buffer_planning_reuses_memory(dev):
    from ratchet_b200 import Tensor, last_resolve_stats
    g = np.random.Generator(np.random.PCG64(3))
    x = Tensor.from_data(g.standard_normal((64, 256)).astype(np.float32), device=dev)
    w = [Tensor.from_data((g.standard_normal((256, 256)) * 0.05).astype(np.float32), device=dev) for _ in range(6)]
    h = x
    for wi in w:                       # matmul cannot run in place: each layer needs a fresh buffer
        h = wi.gemm(h, None, False, True, True).tanh()
    h.resolve()
    st = last_resolve_stats(dev)
    assert st["launched"] == 12 and st["inplace"] == 6
    assert st["buffers"] <= 3          # ping-pong + output, not one per layer
    assert st["planned_bytes"] < st["naive_bytes"]
    ref = x.to_numpy()
    for wi in w:
        ref = np.tanh(ref @ wi.to_numpy().T)
    assert np.allclose(h.to_numpy(), ref, atol=1e-4)


def test_debug_switches_no_reuse_and_profile(dev, capfd):
    """The resolver's debug aids: with no-reuse every tensor gets a buffer of its own and nothing runs in
    place (same results); with profiling every node is bracketed by an event pair and the table names each
    kernel with its count, time and bandwidth."""
    from ratchet_b200 import Tensor, last_resolve_stats
    g = np.random.Generator(np.random.PCG64(31))
    x = g.standard_normal((64, 256)).astype(np.float32)
    w = [(g.standard_normal((256, 256)) * 0.05).astype(np.float32) for _ in range(3)]

    def run():
        h = Tensor.from_data(x, device=dev)
        for wi in w:
            h = Tensor.from_data(wi, device=dev).gemm(h, None, False, True, True).tanh()
        h.resolve()
        return h.to_numpy(), last_resolve_stats(dev)

    base, st0 = run()
    assert st0["inplace"] == 3 and st0["buffers"] <= 3
    dev.set_debug(no_reuse=True, profile=True)
    try:
        dev.profile_report(reset=True)
        again, st1 = run()
        assert st1["inplace"] == 0 and st1["buffers"] == 6 and st1["planned_bytes"] == st1["naive_bytes"]
        assert np.array_equal(again, base)
        table = dev.profile_report(reset=True)
        rows = {ln.split()[0] + " " + ln.split()[1]: ln.split() for ln in table.splitlines()[1:]}
        assert set(rows) == {"matmul f32", "unary f32"}, table
        assert int(rows["matmul f32"][2]) == 3 and int(rows["unary f32"][2]) == 3
        assert float(rows["matmul f32"][3]) > 0 and abs(float(rows["matmul f32"][4]) + float(rows["unary f32"][4]) - 100.0) < 0.2
        assert dev.profile_report() .count("\n") == 1          # cleared
        # the log switch: one line per launching node and a summary per resolve, on stderr
        dev.set_debug(log=True)
        capfd.readouterr()
        run()
        err = capfd.readouterr().err
        assert err.count("[rcu] node") == 6 and "matmul f32 [64, 256]" in err and "unary f32 [64, 256] in place" in err, err
        assert "[rcu] resolve: " in err and "6 launches, 3 in place" in err, err
    finally:
        dev.set_debug()


def test_concat_cache_select_through_graph(dev):
    from ratchet_b200 import Tensor, capi
    g = np.random.Generator(np.random.PCG64(4))
    parts = [g.standard_normal((4, 2, n, 128)).astype(np.float32) for n in (3, 1, 5, 2, 4)]   # ops/concat.rs:290-316
    out = Tensor.cat([Tensor.from_data(p, device=dev) for p in parts], 2)
    assert np.array_equal(out.to_numpy(), np.concatenate(parts, 2))
    cache = Tensor.zeros((1, 2, 16, 8), capi.F32, dev)
    ref_cache = np.zeros((1, 2, 16, 8), np.float32)
    populated = 0
    for n in (3, 1, 1):                # ops/cache.rs:267-302
        src = g.standard_normal((1, 2, n, 8)).astype(np.float32)
        got = cache.cache(Tensor.from_data(src, device=dev), 2, populated).to_numpy()
        ref = orc.cache(ref_cache, src, 2, populated)
        populated += n
        assert np.array_equal(got, ref)
    assert np.array_equal(cache.to_numpy(), ref_cache)
    ids = Tensor.from_data(np.array([[3, 1, 3]], np.int32), device=dev)
    from ratchet_b200 import nn
    table = g.standard_normal((10, 32)).astype(np.float32)
    emb = nn.Embedding(Tensor.from_data(table, device=dev)).schedule(ids)
    assert emb.shape() == (1, 3, 32)
    assert np.array_equal(emb.to_numpy(), table[[3, 1, 3]][None])
    dst = Tensor.from_data(np.array([[1, 2, 3], [4, 5, 6]], np.float32), device=dev)
    wr = dst.index_write(Tensor.from_data(np.array([[7, 8]], np.float32), device=dev), [1, 1])
    assert np.array_equal(wr.to_numpy(), np.array([[1, 2, 3], [4, 7, 8]], np.float32))


# ------------------------------------------------------------------------------ configuration graphs
def test_config1_phi2_mlp_block_f32(dev):
    """x[1,64,2560] -> LayerNorm -> W1[10240,2560]+b1 -> tanh-GELU -> W2[2560,10240]+b2 -> + x, in f32."""
    from ratchet_b200 import Tensor, last_resolve_stats
    W = mb.phi2_mlp_weights(0)
    ref = mb.phi2_mlp_block(OTensor, None, W).schedule(OTensor.from_data(W["x"])).to_numpy()
    out = mb.phi2_mlp_block(Tensor, dev, W).schedule(Tensor.from_data(W["x"], device=dev)).resolve()
    got = out.to_numpy()
    assert got.shape == (1, 64, 2560)
    # five nodes; both projections (80 k-blocks on 80 tiles, 320 k-blocks on 20 tiles) cut K into slices, and each adds
    # the kernel that sums them
    assert last_resolve_stats(dev)["launched"] == 7
    bad = np.abs(got - ref) > 1e-4 + 1e-4 * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} outside 1e-4; max abs {np.abs(got - ref).max():.2e}"


@pytest.mark.parametrize("quant,tol", [("f32", 1e-4), ("q8f", 1e-2), ("q8h", 1e-2)])
def test_config4_whisper_tiny_encoder(dev, quant, tol):
    """mel[1,80,3000] U(-1,1) -> conv stem -> 4 pre-LN blocks (d 384, 6 heads, MLP 1536) -> LayerNorm."""
    from ratchet_b200 import Tensor
    W = mb.whisper_weights(1, quant=quant)
    mel = np.random.Generator(np.random.PCG64(9)).uniform(-1, 1, (1, 80, 3000)).astype(np.float32)
    ref = mb.whisper_encoder(OTensor, None, W).schedule(OTensor.from_data(mel)).full().to_numpy()
    got = mb.whisper_encoder(Tensor, dev, W).schedule(Tensor.from_data(mel, device=dev)).full().to_numpy()
    assert got.shape == (1, 1500, 384)
    bad = np.abs(got - ref) > tol + tol * np.abs(ref)
    assert not bad.any(), f"{quant}: {bad.sum()} of {bad.size} outside {tol}; max abs {np.abs(got - ref).max():.2e}"


@pytest.mark.parametrize("quant,act", [("q8h", np.float16), ("q8f", np.float32)])
def test_config5_phi3_decode_step_two_layers(dev, quant, act):
    """One Phi-3-mini decode step (hidden 3072, 32 heads x 96, MLP 8192, vocab 32064, 1024 prior KV
    positions) with two of the 32 layers, so the oracle finishes in seconds."""
    from ratchet_b200 import Tensor, last_resolve_stats
    W = mb.phi3_weights(2, n_layers=2, quant=quant)
    ids = np.array([[12345]], np.int32)
    ref_model = mb.phi3_model(OTensor, None, W, 1024, act)
    ref = ref_model.schedule(OTensor.from_data(ids)).full().to_numpy()
    model = mb.phi3_model(Tensor, dev, W, 1024, act)
    logits = model.schedule(Tensor.from_data(ids, device=dev)).full().resolve()
    got = logits.to_numpy()
    st = last_resolve_stats(dev)
    assert got.shape == (1, 1, 32064)
    assert st["launched"] > 40
    e = rel_err(got, ref)
    assert e < 1e-2, f"logits differ: normalised max error {e:.3e}"
    assert int(got.argmax()) == int(ref.argmax())
    # the new K/V rows landed in the caches (ops/cache.rs writes the source into the cache too)
    for layer in (0, 1):
        k_dev = model.kv_cache[layer].k_cache.to_numpy()[0, :, 1024]
        k_ref = ref_model.kv_cache[layer].k_cache.to_numpy()[0, :, 1024]
        assert rel_err(k_dev, k_ref) < 1e-2
    model.kv_cache.update(1)
    assert model.kv_cache.entries(0) == 1025
