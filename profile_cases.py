"""One launch group per kernel family at a size that does not fit in L2.

``python profile_cases.py [case ...]`` runs each named case (all of them by default)
``--reps`` times on one GPU, times it with CUDA events on the library's stream and prints one line
per case: microseconds per launch, the algorithmic bytes the launch must move (inputs read once,
outputs written once) and the resulting GB/s, or TFLOP/s for the tensor-core GEMM.  The same command
is the small, self-terminating program to put under a profiler: every case holds well under 2 GB on
the device and launches a handful of kernels.

Inputs are seeded random data produced with numpy here (quantised buffers are filled with random
codes in ratchet's segment layout); no result is checked in this module, the parity tests do that.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

import os

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ratchet_b200 import capi  # noqa: E402


def _rand_f16(rng, n):
    # one gaussian block tiled: host generation of hundreds of MB would dominate the run time
    base = rng.standard_normal(1 << 20).astype(np.float16)
    reps = (n + base.size - 1) // base.size
    return np.tile(base, reps)[:n]


def _q8_buffer(rng, n, dt):
    off = capi.dtype_segments(dt, n)
    buf = np.zeros(capi.dtype_nbytes(dt, n), np.uint8)
    codes = rng.integers(0, 256, 1 << 20, dtype=np.uint8)
    buf[off[0]: off[0] + n] = np.tile(codes, (n + codes.size - 1) // codes.size)[:n]
    if dt == capi.Q8_0F:
        buf[off[1]: off[1] + n // 32 * 4] = np.full(n // 32, 0.0006, np.float32).view(np.uint8)
    else:
        buf[off[1]: off[1] + n // 32 * 2] = np.full(n // 32, 0.0006, np.float16).view(np.uint8)
    return buf


def _q4k_buffer(rng, n):
    nb = n // 256
    off = capi.dtype_segments(capi.Q4_KH, n)
    buf = np.zeros(capi.dtype_nbytes(capi.Q4_KH, n), np.uint8)
    codes = rng.integers(0, 256, 1 << 20, dtype=np.uint8)
    buf[off[0]: off[0] + n // 2] = np.tile(codes, (n // 2 + codes.size - 1) // codes.size)[: n // 2]
    buf[off[1]: off[1] + nb * 12] = np.tile(codes, (nb * 12 + codes.size - 1) // codes.size)[: nb * 12]
    buf[off[2]: off[2] + nb * 2] = np.full(nb, 0.0011, np.float16).view(np.uint8)
    buf[off[3]: off[3] + nb * 2] = np.full(nb, 0.00015, np.float16).view(np.uint8)
    return buf


GEMM_M = 2048     # token rows of the tensor-core GEMM cases (--gemm-m)


class Case:
    """``setup(dev, rng)`` returns (run, algorithmic_bytes, flops_or_None)."""

    def __init__(self, name, setup, kernel, own_graph=False):
        self.name, self.setup, self.kernel = name, setup, kernel
        self.own_graph = own_graph     # the call replays a CUDA graph of its own: it cannot be captured into another


def _elementwise(dev, rng, which):
    n = 64 << 20
    a = dev.from_numpy(_rand_f16(rng, n).reshape(n // 4096, 4096))
    out = dev.empty(capi.F16, a.shape)
    if which == "binary_same":
        b = dev.from_numpy(_rand_f16(rng, n).reshape(a.shape))
        return (lambda: dev.binary("add", a, b, out)), 3 * n * 2, None
    if which == "binary_bcast":
        b = dev.from_numpy(_rand_f16(rng, 4096))
        return (lambda: dev.binary("mul", a, b, out)), 2 * n * 2, None
    if which == "unary_gelu":
        return (lambda: dev.unary("gelu", a, out)), 2 * n * 2, None
    if which == "cast":
        o32 = dev.empty(capi.F32, a.shape)
        return (lambda: dev.cast(a, capi.F32, o32)), n * 6, None
    raise KeyError(which)


def _rows(dev, rng, which):
    if which == "layer_norm":
        rows, N = 65536, 2560
    elif which == "rms_norm":
        rows, N = 65536, 3072
    elif which == "softmax":
        rows, N = 131072, 1500
    elif which == "softmax_long":
        rows, N = 8192, 32064
    else:
        rows, N = 65536, 3072
    x = dev.from_numpy(_rand_f16(rng, rows * N).reshape(rows, N))
    if which in ("layer_norm", "rms_norm"):
        g = dev.from_numpy(_rand_f16(rng, N))
        b = dev.from_numpy(_rand_f16(rng, N)) if which == "layer_norm" else None
        out = dev.empty(capi.F16, x.shape)
        kind = capi.LAYER_NORM if which == "layer_norm" else capi.RMS_NORM
        return (lambda: dev.norm(kind, x, g, b, 1e-5, 0, out)), 2 * rows * N * 2, None
    if which.startswith("softmax"):
        out = dev.empty(capi.F16, x.shape)
        return (lambda: dev.softmax(x, 1, out)), 2 * rows * N * 2, None
    out = dev.empty(capi.F16, (rows,))
    return (lambda: dev.reduce(capi.REDUCE_SUM, x, out)), rows * N * 2, None


def _rope(dev, rng):
    shape = (8, 32, 4096, 96)
    n = int(np.prod(shape))
    x = dev.from_numpy(_rand_f16(rng, n).reshape(shape))
    out = dev.empty(capi.F16, shape)
    return (lambda: dev.rope(x, 96, 10000.0, 0, out)), 2 * n * 2, None


def _reindex(dev, rng, which):
    if which == "permute":
        shape = (8, 4096, 32, 96)
        n = int(np.prod(shape))
        x = dev.from_numpy(_rand_f16(rng, n).reshape(shape))
        out = dev.empty(capi.F16, (8, 32, 4096, 96))
        return (lambda: dev.permute(x, (0, 2, 1, 3), out)), 2 * n * 2, None
    if which == "transpose":
        R, Cc = 16384, 8192
        x = dev.from_numpy(_rand_f16(rng, R * Cc).reshape(R, Cc))
        out = dev.empty(capi.F16, (Cc, R))
        return (lambda: dev.permute(x, (1, 0), out)), 2 * R * Cc * 2, None
    if which == "concat":
        a = dev.from_numpy(_rand_f16(rng, 32 * 4096 * 256).reshape(32, 4096, 256))
        b = dev.from_numpy(_rand_f16(rng, 32 * 4096 * 256).reshape(32, 4096, 256))
        out = dev.empty(capi.F16, (32, 8192, 256))
        return (lambda: dev.concat([a, b], 1, out)), 2 * 2 * a.numel * 2, None
    if which == "slice":
        x = dev.from_numpy(_rand_f16(rng, 32 * 8192 * 256).reshape(32, 8192, 256))
        out = dev.empty(capi.F16, (32, 4096, 256))
        return (lambda: dev.slice(x, [(0, 32), (1024, 5120), (0, 256)], out)), 2 * out.numel * 2, None
    if which == "broadcast":
        x = dev.from_numpy(_rand_f16(rng, 4096).reshape(1, 4096))
        out = dev.empty(capi.F16, (32768, 4096))
        return (lambda: dev.broadcast(x, (32768, 4096), out)), out.numel * 2, None
    if which == "index_select":
        table = dev.from_numpy(_rand_f16(rng, 32064 * 3072).reshape(32064, 3072))
        ids = dev.from_numpy(rng.integers(0, 32064, 32768).astype(np.int32))
        out = dev.empty(capi.F16, (32768, 3072))
        return (lambda: dev.index_select(table, ids, 0, out)), 2 * out.numel * 2, None
    if which == "index_select_q8":
        n = 32064 * 3072
        table = dev.from_quantized(_q8_buffer(rng, n, capi.Q8_0H), capi.Q8_0H, (32064, 3072))
        ids = dev.from_numpy(rng.integers(0, 32064, 32768).astype(np.int32))
        out = dev.empty(capi.F16, (32768, 3072))
        return (lambda: dev.index_select(table, ids, 0, out)), out.numel * 2 + out.numel * (1 + 2 / 32), None
    raise KeyError(which)


def _conv(dev, rng):
    B, Cin, L, Cout = 32, 384, 3000, 384
    x = dev.from_numpy(_rand_f16(rng, B * Cin * L).astype(np.float32).reshape(B, Cin, L))
    w = dev.from_numpy((_rand_f16(rng, Cout * Cin * 3).astype(np.float32) * 0.02).reshape(Cout, Cin, 3))
    b = dev.from_numpy(np.zeros(Cout, np.float32))
    out = dev.empty(capi.F32, (B, Cout, 1500))
    flops = 2.0 * B * Cout * 1500 * Cin * 3
    return (lambda: dev.conv1d(x, w, b, 2, 1, out)), (x.numel + out.numel + w.numel) * 4, flops


def _dequant(dev, rng, which):
    n = 128 << 20
    if which == "dequant_q8":
        src = dev.from_quantized(_q8_buffer(rng, n, capi.Q8_0H), capi.Q8_0H, (n // 4096, 4096))
        nbytes = n + n // 16 + 2 * n
    else:
        src = dev.from_quantized(_q4k_buffer(rng, n), capi.Q4_KH, (n // 4096, 4096))
        nbytes = n // 256 * 144 + 2 * n
    out = dev.empty(capi.F16, (n // 4096, 4096))
    return (lambda: dev.dequantize(src, out)), nbytes, None


def _gemv(dev, rng, which):
    N, K = 16384, 16384
    x = dev.from_numpy(_rand_f16(rng, K).reshape(1, K))
    out = dev.empty(capi.F16, (1, N))
    if which == "gemv_f16":
        w = dev.from_numpy((_rand_f16(rng, N * K).astype(np.float32) * 0.02).astype(np.float16).reshape(N, K))
        nbytes = N * K * 2
    elif which == "gemv_q4k":
        w = dev.from_quantized(_q4k_buffer(rng, N * K), capi.Q4_KH, (N, K))
        nbytes = N * K // 2 + N * K // 256 * 16
    else:
        w = dev.from_quantized(_q8_buffer(rng, N * K, capi.Q8_0H), capi.Q8_0H, (N, K))
        nbytes = N * K + N * K // 16
    return (lambda: dev.matmul(w, x, None, False, True, True, out)), nbytes + K * 2 + N * 2, None


def _gemm(dev, rng, which):
    if which == "gemm_simt_f32":
        M, N, K = 64, 10240, 2560
        w = dev.from_numpy((_rand_f16(rng, N * K).astype(np.float32) * 0.02).reshape(N, K))
        x = dev.from_numpy(_rand_f16(rng, M * K).astype(np.float32).reshape(M, K))
        out = dev.empty(capi.F32, (M, N))
        return (lambda: dev.matmul(w, x, None, False, True, True, out)), (N * K + M * K + M * N) * 4, 2.0 * M * N * K
    M, N, K = GEMM_M, 8192, 3072
    if which == "gemm_tc_f32":
        w = dev.from_numpy((_rand_f16(rng, N * K).astype(np.float32) * 0.02).reshape(N, K))
        x = dev.from_numpy(_rand_f16(rng, M * K).astype(np.float32).reshape(M, K))
        out = dev.empty(capi.F32, (M, N))
        return (lambda: dev.matmul(w, x, None, False, True, True, out)), (N * K + M * K + M * N) * 4, 2.0 * M * N * K
    x = dev.from_numpy(_rand_f16(rng, M * K).reshape(M, K))
    out = dev.empty(capi.F16, (M, N))
    if which == "gemm_tc_f16":
        w = dev.from_numpy((_rand_f16(rng, N * K).astype(np.float32) * 0.02).astype(np.float16).reshape(N, K))
        nbytes = N * K * 2
    elif which == "gemm_tc_q8":
        w = dev.from_quantized(_q8_buffer(rng, N * K, capi.Q8_0H), capi.Q8_0H, (N, K))
        nbytes = N * K + N * K // 16
    else:
        w = dev.from_quantized(_q4k_buffer(rng, N * K), capi.Q4_KH, (N, K))
        nbytes = N * K // 256 * 144
    return (lambda: dev.matmul(w, x, None, False, True, True, out)), nbytes + (M * K + M * N) * 2, 2.0 * M * N * K


def _attention(dev, rng):
    H, hd, max_cache, P = 32, 96, 4096, 4000
    qkv = dev.from_numpy(_rand_f16(rng, 3 * H * hd))
    kc = dev.from_numpy(_rand_f16(rng, H * max_cache * hd).reshape(H, max_cache, hd))
    vc = dev.from_numpy(_rand_f16(rng, H * max_cache * hd).reshape(H, max_cache, hd))
    out = dev.empty(capi.F16, (H * hd,))
    lib = dev._lib

    def run():
        dev.check(lib.rcu_attn_decode(dev.handle, qkv.ptr, kc.ptr, vc.ptr, H, H, hd, max_cache, hd, 10000.0, P, out.ptr))
    return run, 2 * H * (P + 1) * hd * 2, None


def _decode_step(dev, rng):
    """The data-flow decode kernel on a four-layer model of Phi-3-mini's width (hidden 3072, 32 heads x 96,
    MLP 8192, vocabulary 32064, Q8_0H, 1024 cached positions): per layer the same jobs as the 32-layer
    step of the benchmark, small enough (0.7 GB) for a multi-pass capture."""
    from ratchet_b200.decoder import Decoder, DecoderConfig, DecoderLayer
    L, d, H, hd, ffn, V, cache, prior = 4, 3072, 32, 96, 8192, 32064, 4096, 1024

    def q8h(N, K):
        buf = np.zeros(capi.dtype_nbytes(capi.Q8_0H, N * K), np.uint8)
        rows = min(N, 512)
        q = rng.integers(-127, 128, (rows, K), dtype=np.int8)
        sc = (np.abs(rng.standard_normal((rows, K // 32))) * 0.0004 + 0.0003).astype(np.float16)
        off = capi.dtype_segments(capi.Q8_0H, N * K)[1]
        qs = buf[: N * K].view(np.int8).reshape(N, K)
        ds = buf[off: off + (N * K // 32) * 2].view(np.float16).reshape(N, K // 32)
        for r0 in range(0, N, rows):
            n = min(rows, N - r0)
            qs[r0: r0 + n] = q[:n]
            ds[r0: r0 + n] = sc[:n]
        return buf

    shapes = {"qkv": (3 * H * hd, d), "o": (d, d), "up": (2 * ffn, d), "down": (d, ffn)}
    host = {k: q8h(*v) for k, v in shapes.items()}
    kv = np.zeros((H, cache, hd), np.float16)
    kv[:, :prior] = rng.standard_normal((H, prior, hd)).astype(np.float16)
    ones = np.ones(d, np.float32)
    layers = [DecoderLayer(dev.from_numpy(ones), dev.from_quantized(host["qkv"], capi.Q8_0H, shapes["qkv"]),
                           dev.from_quantized(host["o"], capi.Q8_0H, shapes["o"]), dev.from_numpy(ones),
                           dev.from_quantized(host["up"], capi.Q8_0H, shapes["up"]), dev.from_quantized(host["down"], capi.Q8_0H, shapes["down"]),
                           dev.from_numpy(kv), dev.from_numpy(kv)) for _ in range(L)]
    emb = dev.from_quantized(q8h(V, d), capi.Q8_0H, (V, d))
    head = dev.from_quantized(q8h(V, d), capi.Q8_0H, (V, d))
    cfg = DecoderConfig(L, d, H, H, hd, ffn, V, cache, hd, 10000.0, 1e-5, capi.Q8_0H)
    dec = Decoder(dev, cfg, layers, emb, dev.from_numpy(ones), head)
    token = dev.from_numpy(np.array([17], np.int32))
    logits = dev.empty(capi.F16, (V,))
    import ctypes as C

    def run():
        dec.position = prior
        dev.check(dev._lib.rcu_decoder_step(dec._h, C.c_void_p(token.ptr), C.c_void_p(logits.ptr), None))
    w_elems = L * (4 * d * d + 3 * ffn * d) + V * d
    return run, int(w_elems * 1.0625) + L * 2 * H * (prior + 1) * hd * 2, None


CASES = [
    Case("binary_same", lambda d, r: _elementwise(d, r, "binary_same"), "binary_same_kernel"),
    Case("binary_bcast", lambda d, r: _elementwise(d, r, "binary_bcast"), "binary_bcast_kernel"),
    Case("unary_gelu", lambda d, r: _elementwise(d, r, "unary_gelu"), "unary_kernel"),
    Case("cast", lambda d, r: _elementwise(d, r, "cast"), "cast_kernel"),
    Case("layer_norm", lambda d, r: _rows(d, r, "layer_norm"), "row_kernel"),
    Case("rms_norm", lambda d, r: _rows(d, r, "rms_norm"), "row_kernel"),
    Case("softmax", lambda d, r: _rows(d, r, "softmax"), "row_kernel"),
    Case("softmax_long", lambda d, r: _rows(d, r, "softmax_long"), "row_kernel_long"),
    Case("reduce_sum", lambda d, r: _rows(d, r, "reduce"), "reduce_rows_kernel"),
    Case("rope", _rope, "rope_kernel"),
    Case("permute", lambda d, r: _reindex(d, r, "permute"), "remap4_kernel"),
    Case("transpose", lambda d, r: _reindex(d, r, "transpose"), "transpose_kernel"),
    Case("concat", lambda d, r: _reindex(d, r, "concat"), "copy2d_kernel"),
    Case("slice", lambda d, r: _reindex(d, r, "slice"), "copy2d_kernel / remap4_kernel"),
    Case("broadcast", lambda d, r: _reindex(d, r, "broadcast"), "remap4_kernel"),
    Case("index_select", lambda d, r: _reindex(d, r, "index_select"), "gather_kernel"),
    Case("index_select_q8", lambda d, r: _reindex(d, r, "index_select_q8"), "gather_q8_kernel"),
    Case("conv1d", _conv, "conv1d_k3_kernel"),
    Case("dequant_q8", lambda d, r: _dequant(d, r, "dequant_q8"), "dequant_q8_kernel"),
    Case("dequant_q4k", lambda d, r: _dequant(d, r, "dequant_q4k"), "dequant_q4k_kernel"),
    Case("gemv_f16", lambda d, r: _gemv(d, r, "gemv_f16"), "gemv_float_kernel"),
    Case("gemv_q8", lambda d, r: _gemv(d, r, "gemv_q8"), "gemv_q8_ring_kernel"),
    Case("gemv_q4k", lambda d, r: _gemv(d, r, "gemv_q4k"), "gemv_q4k_kernel"),
    Case("gemm_f32_phi2_mlp", lambda d, r: _gemm(d, r, "gemm_simt_f32"), "gemm_tc_f32_kernel (M=64, N=10240, K=2560)"),
    Case("gemm_tc_f32", lambda d, r: _gemm(d, r, "gemm_tc_f32"), "gemm_tc_f32_kernel"),
    Case("gemm_tc_f16", lambda d, r: _gemm(d, r, "gemm_tc_f16"), "gemm_tc2_kernel"),
    Case("gemm_tc_q8", lambda d, r: _gemm(d, r, "gemm_tc_q8"), "gemm_tc_kernel"),
    Case("gemm_tc_q4k", lambda d, r: _gemm(d, r, "gemm_tc_q4k"), "gemm_tc_kernel"),
    Case("attn_decode", _attention, "attn_decode_kernel"),
    Case("decode_step", _decode_step, "decode_flow_kernel (4 layers of Phi-3-mini width + lm_head)", own_graph=True),
]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("cases", nargs="*", help="case names (default: all); --list shows them")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--reps", type=int, default=10, help="launches per case captured into one CUDA graph (after one eager warm-up)")
    ap.add_argument("--replays", type=int, default=3, help="timed replays of that graph")
    ap.add_argument("--gemm-m", type=int, default=2048, help="token rows M of the gemm_tc_* cases")
    args = ap.parse_args(argv)
    global GEMM_M
    GEMM_M = args.gemm_m
    if args.list:
        for c in CASES:
            print(f"{c.name:18s} {c.kernel}")
        return 0
    by_name = {c.name: c for c in CASES}
    unknown = [n for n in args.cases if n not in by_name]
    if unknown:
        ap.error(f"unknown case(s) {unknown}; --list shows the names")
    chosen = [by_name[n] for n in args.cases] if args.cases else CASES

    import torch
    from ratchet_b200.device import Device
    if not torch.cuda.is_available():
        print("profile_cases needs a CUDA device (there is no CPU path)", file=sys.stderr)
        return 2
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)       # graph replays and events below all go to the library's stream
    dev = Device(0, stream=stream.cuda_stream)
    peak = None
    try:
        import os
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peak = json.load(f)
    except Exception:
        pass
    for c in chosen:
        rng = np.random.Generator(np.random.PCG64(1234))
        run, nbytes, flops = c.setup(dev, rng)
        l0 = dev.launches
        run()
        per_call = dev.launches - l0
        stream.synchronize()
        # the timed launches replay from a CUDA graph, so host time per call is out of the picture
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if c.own_graph:
            run()                      # the second call is the first graph replay
            e0.record(stream)
            for _ in range(args.reps * args.replays):
                run()
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(args.reps):
                    run()
            e0.record(stream)
            for _ in range(args.replays):
                graph.replay()
        e1.record(stream)
        stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (args.reps * args.replays)
        rec = {"case": c.name, "kernel": c.kernel, "launches_per_call": per_call, "us": round(us, 2),
               "algorithmic_bytes": int(nbytes), "gbs": round(nbytes / us * 1e-3, 1)}
        if peak:
            rec["frac_of_measured_hbm"] = round(rec["gbs"] / peak["hbm_gbs"], 3)
        if flops:
            rec["tflops"] = round(flops / us * 1e-6, 1)
        print(json.dumps(rec), flush=True)
        del run
        import gc
        gc.collect()
    dev.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
