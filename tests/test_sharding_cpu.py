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
from ratchet_b200.comm import exchange_handles, shard_q8, shard_rows


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
