"""Host-side logic of the row-sharded Linear, without a GPU: shard layout of ratchet Q8_0 buffers and
the handle exchange / gather plumbing over torch.distributed (gloo, world size 2)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc
from ratchet_b200 import capi
from ratchet_b200.comm import decoder_shard_ranges, exchange_handles, shard_q8, shard_rows, take_rows_q8


def test_shard_rows():
    assert [shard_rows(65536, r, 8) for r in (0, 7)] == [(0, 8192), (57344, 65536)]
    with pytest.raises(ValueError):
        shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_q8_is_a_ratchet_buffer_of_the_rows(half, world):
    g = np.random.Generator(np.random.PCG64(world))
    N, K = 64, 96
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float16 if half else np.float32)
    x = g.standard_normal(K).astype(np.float16)
    full = orc.quantize_q8(w)
    dt = capi.Q8_0H if half else capi.Q8_0F
    y_full = orc.gemv_q8(full, N, K, half, x)
    parts = []
    for r in range(world):
        sh = shard_q8(full, dt, N, K, r, world)
        r0, r1 = shard_rows(N, r, world)
        assert sh.size == orc.q8_nbytes((r1 - r0) * K, half)
        # a shard is exactly what quantising the row slice alone produces
        assert np.array_equal(sh, orc.quantize_q8(w[r0:r1]))
        parts.append(orc.gemv_q8(sh, r1 - r0, K, half, x))
    assert np.array_equal(np.concatenate(parts).view(np.uint16), y_full.view(np.uint16))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = np.random.Generator(np.random.PCG64(0))
        N, K = 128, 64
        w = (g.standard_normal((N, K)) * 0.02).astype(np.float32)
        x = g.standard_normal(K).astype(np.float16)
        full = orc.quantize_q8(w)
        # handle exchange: every rank sees every rank's 64 bytes in rank order
        mine = bytes([rank]) * 64
        handles = exchange_handles(mine, rank, world)
        assert handles == [bytes([r]) * 64 for r in range(world)]
        # shard, compute the local slice with the oracle, gather: equals the unsharded result
        sh = shard_q8(full, capi.Q8_0F, N, K, rank, world)
        y_local = torch.from_numpy(orc.gemv_q8(sh, N // world, K, False, x).view(np.uint8).copy())
        out = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(out, y_local)
        y = torch.cat(out).numpy().view(np.float16)
        ref = orc.gemv_q8(full, N, K, False, x)
        q.put((rank, bool(np.array_equal(y.view(np.uint16), ref.view(np.uint16)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_decoder_shards_cover_every_row_once(world):
    """Sharded decode step: the union of the ranks' row ranges is every output row exactly once, the
    qkv shard holds the q, k and v rows of the rank's own heads, gate and up rows pair up."""
    H, Hkv, hd, d, ffn, vocab = 32, 32, 96, 3072, 8192, 32064
    seen = {k: np.zeros(n, np.int32) for k, n in (("qkv", (H + 2 * Hkv) * hd), ("o", d), ("gate_up", 2 * ffn), ("down", d), ("lm_head", vocab))}
    for r in range(world):
        R = decoder_shard_ranges(H, Hkv, hd, d, ffn, vocab, r, world)
        for k, cnt in seen.items():
            for a, b in R[k]:
                cnt[a:b] += 1
        (q0, q1), (k0, k1), (v0, v1) = R["qkv"]
        assert q1 - q0 == H // world * hd and k1 - k0 == v1 - v0 == Hkv // world * hd
        assert k0 - H * hd == v0 - (H + Hkv) * hd == R["kv_heads"][0] * hd          # k and v rows of the same heads
        (g0, g1), (u0, u1) = R["gate_up"]
        assert u0 - g0 == ffn and u1 - g1 == ffn                                     # up row = gate row + ffn
    assert all((c == 1).all() for c in seen.values())
    with pytest.raises(ValueError):
        decoder_shard_ranges(32, 32, 96, 3072, 8192, 32064, 0, 5)


def test_take_rows_q8_concatenates_ranges():
    g = np.random.Generator(np.random.PCG64(3))
    N, K = 48, 64
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float16)
    full = orc.quantize_q8(w)
    sub = take_rows_q8(full, capi.Q8_0H, N, K, [(8, 16), (40, 48)])
    picked = np.concatenate([w[8:16], w[40:48]])
    assert np.array_equal(sub, orc.quantize_q8(picked))
    assert np.array_equal(orc.dequantize_q8(sub, (16, K), True).view(np.uint16),
                          np.concatenate([orc.dequantize_q8(full, (N, K), True)[8:16], orc.dequantize_q8(full, (N, K), True)[40:48]]).view(np.uint16))
    with pytest.raises(ValueError):
        take_rows_q8(full, capi.Q8_0H, N, K, [(40, 49)])


def test_two_rank_gather_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=10) for _ in range(world))
    assert results == [(0, True), (1, True)]
