"""ane_b200 -- the maderix/ANE per-layer non-matmul operator set on NVIDIA B200.

``ane_b200.lib``      ctypes binding of libane_cuda.so (the C ABI of include/ane_cuda.h)
``ane_b200.cpu_ops``  the reference's operator interface (same names and arguments) on host arrays
``ane_b200.dev_ops``  the device-resident operators on torch CUDA tensors
``ane_b200.sharded``  token sharding and the collectives around the operators (multi-GPU)
"""
from . import lib  # noqa: F401

__all__ = ["lib"]
