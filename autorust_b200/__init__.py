"""autorust_b200 -- autorust's fused attention path as hand-written sm_100a kernels.

The package holds the CUDA sources and their C ABI (csrc/, built into lib/ by build.py), ctypes
bindings (_abi.py), torch-facing call wrappers (ops.py) and the host-side mirror of autorust's
Tensor / Session / Settings attention surface (host.py over csrc/host/).
"""
from . import _abi  # noqa: F401

__all__ = ["_abi"]
