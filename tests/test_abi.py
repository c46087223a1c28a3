"""The C-ABI shared library loads and exports every symbol include/ratchet_cuda.h declares, and the
ctypes table binds exactly that set.  No compute call is made (this runs without a GPU)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ratchet_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rcu_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    import __graft_entry__ as entry
    entry.build()
    from ratchet_b200 import capi
    names = declared_symbols()
    assert len(names) > 30
    handle = ctypes.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"
    assert sorted(capi.SIGNATURES) == names, set(capi.SIGNATURES) ^ set(names)
    capi.lib()


def test_layout_queries_without_gpu():
    from oracle import oracle as orc
    from ratchet_b200 import capi
    # dtype/blocks.rs:69-82,124-148 through the C ABI (pure host arithmetic)
    n = 65536 * 16384
    assert capi.dtype_nbytes(capi.Q8_0F, n) == 1073741824 + 134217728 == orc.q8_nbytes(n, False)
    n = 9216 * 3072
    assert capi.dtype_nbytes(capi.Q8_0H, n) == 28311552 + 1769472
    n = 8192 * 3072
    assert capi.dtype_nbytes(capi.Q4_KH, n) == 14155776
    assert capi.dtype_segments(capi.Q4_KH, n) == orc.q4k_offsets(n, True)
    assert capi.dtype_nbytes(capi.F32, 1) == 16 and capi.dtype_nbytes(capi.F16, 9) == 20   # min 16 B, 4-B multiple
    assert capi.activation_dtype(capi.Q8_0H) == capi.F16 and capi.activation_dtype(capi.Q4_KF) == capi.F32


def test_opening_a_device_without_gpu_fails_loudly():
    import pytest
    import torch
    from ratchet_b200 import Device, RatchetCudaError
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RatchetCudaError):
        Device(0)
