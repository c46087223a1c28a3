"""GGUF reader and transcoder without a GPU: files written here in the public GGUF container format
(v1, v2 and v3 headers) with F32 / F16 / Q8_0 / Q4_K tensors whose ggml blocks are built from the
oracle's quantisers; the transcoded buffers must be byte-identical with the oracle's ratchet buffers,
including the edge codes (-128 in Q8_0, all-ones nibbles and 6-bit codes in Q4_K)."""
import struct

import numpy as np
import pytest

from oracle import oracle as orc
from ratchet_b200 import capi
from ratchet_b200.capi import RatchetCudaError
from ratchet_b200.gguf import GGML_F16, GGML_F32, GGML_Q4_K, GGML_Q8_0, GGUFFile


def _s(text, version):
    b = text.encode()
    return (struct.pack("<I", len(b)) if version == 1 else struct.pack("<Q", len(b))) + b


def _n(v, version):
    return struct.pack("<I", v) if version == 1 else struct.pack("<Q", v)


def write_gguf(path, tensors, meta, version=3, alignment=None):
    """tensors: list of (name, shape in ratchet order, ggml_type, raw bytes); meta: list of (key, type id, packed value)."""
    kv = list(meta)
    if alignment is not None:
        kv.append(("general.alignment", 4, struct.pack("<I", alignment)))
    head = struct.pack("<II", 0x46554747, version) + _n(len(tensors), version) + _n(len(kv), version)
    for key, vt, payload in kv:
        head += _s(key, version) + struct.pack("<I", vt) + payload
    align = alignment or 32
    offsets, data = [], b""
    for _, _, _, raw in tensors:
        data += b"\0" * (-len(data) % align)
        offsets.append(len(data))
        data += raw
    for (name, shape, gt, _), off in zip(tensors, offsets):
        head += _s(name, version) + struct.pack("<I", len(shape))
        for d in reversed(shape):                      # innermost first on disk
            head += _n(d, version)
        head += struct.pack("<IQ", gt, off)
    head += b"\0" * (-len(head) % align)
    with open(path, "wb") as f:
        f.write(head + data)


def ggml_q8_0_blocks(ratchet_q8h, numel):
    """ratchet Q8_0H buffer -> ggml block_q8_0 stream {f16 d; i8 qs[32]}."""
    off = capi.dtype_segments(capi.Q8_0H, numel)
    qs = ratchet_q8h[off[0]: off[0] + numel].reshape(-1, 32)
    d = ratchet_q8h[off[1]: off[1] + numel // 32 * 2].reshape(-1, 2)
    return np.concatenate([d, qs], axis=1).tobytes()


def ggml_q4_k_blocks(ratchet_q4kh, numel):
    """ratchet Q4_KH buffer -> ggml block_q4_K stream {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]}."""
    nb = numel // 256
    off = capi.dtype_segments(capi.Q4_KH, numel)
    qs = ratchet_q4kh[off[0]: off[0] + nb * 128].reshape(nb, 128)
    sc = ratchet_q4kh[off[1]: off[1] + nb * 12].reshape(nb, 12)
    dmin = ratchet_q4kh[off[2]: off[2] + nb * 2].reshape(nb, 2)
    d = ratchet_q4kh[off[3]: off[3] + nb * 2].reshape(nb, 2)
    return np.concatenate([d, dmin, sc, qs], axis=1).tobytes()


@pytest.mark.parametrize("version", [1, 2, 3])
def test_transcode_matches_the_oracle_layout(tmp_path, version):
    g = np.random.Generator(np.random.PCG64(version))
    w8 = (g.standard_normal((48, 64)) * 0.02).astype(np.float16)
    q8h = orc.quantize_q8(w8)
    q8h[5] = 0x80                                           # the -128 code ggml never writes but the layout admits
    w4 = (g.standard_normal((6, 512)) * 0.02).astype(np.float32)
    q4h = orc.quantize_q4k(w4, True)
    off4 = capi.dtype_segments(capi.Q4_KH, w4.size)
    q4h[off4[0]: off4[0] + 16] = 0xFF                       # all-ones nibbles
    q4h[off4[1]: off4[1] + 12] = 0xFF                       # all-ones 6-bit scale / min codes
    f32 = g.standard_normal((3, 5, 7)).astype(np.float32)
    f16 = g.standard_normal((9,)).astype(np.float16)
    path = str(tmp_path / f"v{version}.gguf")
    write_gguf(path, [("blk.0.attn_qkv.weight", (48, 64), GGML_Q8_0, ggml_q8_0_blocks(q8h, w8.size)),
                      ("blk.0.ffn_up.weight", (6, 512), GGML_Q4_K, ggml_q4_k_blocks(q4h, w4.size)),
                      ("pos", (3, 5, 7), GGML_F32, f32.tobytes()), ("bias", (9,), GGML_F16, f16.tobytes())],
               [("general.architecture", 8, _s("phi3", version)), ("phi3.block_count", 4, struct.pack("<I", 32)),
                ("phi3.attention.layer_norm_rms_epsilon", 6, struct.pack("<f", 1e-5)),
                ("tokenizer.ggml.tokens", 9, struct.pack("<I", 8) + _n(2, version) + _s("a", version) + _s("bc", version)),
                ("some.ints", 9, struct.pack("<I", 5) + _n(3, version) + struct.pack("<iii", 1, 2, 3))],
               version=version, alignment=64 if version == 3 else None)
    with GGUFFile(path) as f:
        assert f.version == version
        assert list(f.tensors) == ["blk.0.attn_qkv.weight", "blk.0.ffn_up.weight", "pos", "bias"]
        assert f.tensors["pos"].shape == (3, 5, 7) and f.tensors["blk.0.attn_qkv.weight"].shape == (48, 64)
        assert f.meta_str("general.architecture") == "phi3" and f.meta_int("phi3.block_count") == 32
        assert abs(f.meta_float("phi3.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
        # f16-capable device: f16 scales, bytes identical with the oracle's buffers
        assert f.target_dtype("blk.0.attn_qkv.weight", True) == capi.Q8_0H
        assert np.array_equal(f.transcode("blk.0.attn_qkv.weight"), q8h)
        assert np.array_equal(f.transcode("blk.0.ffn_up.weight"), q4h)
        # f32 device: scales widened exactly (dtype.rs:139-141 `block.d.to_f32()`)
        assert f.target_dtype("blk.0.attn_qkv.weight", False) == capi.Q8_0F
        q8f = f.transcode("blk.0.attn_qkv.weight", capi.Q8_0F)
        off8h, off8f = capi.dtype_segments(capi.Q8_0H, w8.size), capi.dtype_segments(capi.Q8_0F, w8.size)
        nblk = w8.size // 32
        assert np.array_equal(q8f[: w8.size], q8h[: w8.size])
        assert np.array_equal(q8f[off8f[1]: off8f[1] + nblk * 4].view(np.float32),
                              q8h[off8h[1]: off8h[1] + nblk * 2].view(np.float16).astype(np.float32))
        q4f = f.transcode("blk.0.ffn_up.weight", capi.Q4_KF)
        off4f = capi.dtype_segments(capi.Q4_KF, w4.size)
        nb = w4.size // 256
        assert np.array_equal(q4f[off4f[3]: off4f[3] + nb * 4].view(np.float32), q4h[off4[3]: off4[3] + nb * 2].view(np.float16).astype(np.float32))
        assert np.array_equal(q4f[: nb * 128], q4h[: nb * 128])
        assert np.array_equal(f.transcode("pos"), f32) and np.array_equal(f.transcode("bias").view(np.uint16), f16.view(np.uint16))
        with pytest.raises(RatchetCudaError):
            f.transcode("pos", capi.Q8_0H)


def test_rejects_what_the_reference_rejects(tmp_path):
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 60)
    with pytest.raises(RatchetCudaError) as e:
        GGUFFile(str(bad))
    assert "not a GGUF" in str(e.value)
    # an unsupported ggml dtype can be listed but not loaded (gguf.rs:156); a block-size mismatch is an error (gguf.rs:119-123)
    path = str(tmp_path / "odd.gguf")
    write_gguf(path, [("q6", (256,), 14, b"\0" * 210), ("short", (40,), GGML_Q8_0, b"\0" * 34)], [])
    with GGUFFile(path) as f:
        assert f.tensors["q6"].ggml_type == 14
        with pytest.raises(RatchetCudaError) as e1:
            f.transcode("q6")
        assert "unsupported ggml dtype" in str(e1.value)
        with pytest.raises(RatchetCudaError) as e2:
            f.transcode("short", capi.Q8_0H)
        assert "not divisible by the block size" in str(e2.value)
    # truncated data section
    trunc = tmp_path / "trunc.gguf"
    write_gguf(str(trunc), [("w", (64,), GGML_F32, b"\0" * 256)], [])
    raw = trunc.read_bytes()
    trunc.write_bytes(raw[:-100])
    with GGUFFile(str(trunc)) as f:
        with pytest.raises(RatchetCudaError):
            f.transcode("w")


def test_hostile_lengths_are_refused_not_followed(tmp_path):
    """Lengths, counts and offsets come from the file: values chosen so that `position + length` wraps around
    64 bits must be refused like any other value that points outside the file."""
    huge = 0xFFFFFFFFFFFFFFF0
    # a metadata string whose length wraps position + length
    p1 = tmp_path / "str.gguf"
    p1.write_bytes(struct.pack("<II", 0x46554747, 3) + struct.pack("<QQ", 0, 1) + struct.pack("<Q", huge) + b"k" * 64)
    with pytest.raises(RatchetCudaError):
        GGUFFile(str(p1))
    # an array of u64 whose count times the element size wraps
    p2 = tmp_path / "arr.gguf"
    p2.write_bytes(struct.pack("<II", 0x46554747, 3) + struct.pack("<QQ", 0, 1) + _s("a", 3) + struct.pack("<I", 9) +
                   struct.pack("<I", 10) + struct.pack("<Q", 0x2000000000000001) + b"\0" * 64)
    with pytest.raises(RatchetCudaError):
        GGUFFile(str(p2))
    # a tensor whose shape overflows the element count, and one whose offset wraps data_offset + offset
    p3 = tmp_path / "shape.gguf"
    p3.write_bytes(struct.pack("<II", 0x46554747, 3) + struct.pack("<QQ", 1, 0) + _s("w", 3) + struct.pack("<I", 2) +
                   struct.pack("<QQ", 1 << 40, 1 << 40) + struct.pack("<IQ", GGML_F32, 0) + b"\0" * 64)
    with pytest.raises(RatchetCudaError) as e:
        GGUFFile(str(p3))
    assert "impossible shape" in str(e.value)
    p4 = str(tmp_path / "off.gguf")
    write_gguf(p4, [("w", (64,), GGML_F32, b"\0" * 256)], [])
    raw = bytearray(open(p4, "rb").read())
    at = raw.index(b"w") + 1 + 4 + 8 + 4          # name, rank, one dimension, type -> the offset field
    raw[at: at + 8] = struct.pack("<Q", huge)
    open(p4, "wb").write(bytes(raw))
    with GGUFFile(p4) as f:
        with pytest.raises(RatchetCudaError) as e:
            f.transcode("w")
        assert "past the end of the file" in str(e.value)
