"""bnk_b200 -- the bnk dataplane hot path on B200 (sm_100a).

Batched WireGuard transport-data seal/open, send counters, anti-replay window and
the ACL packet filter, implemented as CUDA kernels in libbnkgpu.so (C ABI in
include/bnk_gpu.h).  The Python modules here only bind that library and mirror the
reference's Go interfaces for tests and benchmarks; nothing computes on the CPU.
"""
from . import _lib  # noqa: F401
from .device import Batch, Context, slot_size  # noqa: F401

__all__ = ["Batch", "Context", "slot_size"]
