"""ratchet_b200 — an sm_100a CUDA device for ratchet-core's tensor-op hot path.

The package is a thin host-side mirror of the reference's Device / Tensor interface over the C ABI
in ``include/ratchet_cuda.h``.  All computation happens in ``libratchet_cuda.so``; importing the
package never computes anything on the host, and opening a device fails loudly when the library
or a B200 is missing.
"""
from . import capi
from .capi import RatchetCudaError
from .device import Buffer, Device
from .tensor import Tensor, last_resolve_stats

__all__ = ["capi", "Buffer", "Device", "RatchetCudaError", "Tensor", "last_resolve_stats"]
