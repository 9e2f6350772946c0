"""B200 (sm_100a) implementation of zdraw's DiT joint-attention path behind a C ABI.

``mattn`` mirrors the reference's operator interface; ``_lib`` is the ctypes binding of
``libzdraw_cuda.so`` (built from ``csrc/``); ``workloads`` holds the synthetic configurations.
"""
from . import _lib, mattn, workloads  # noqa: F401
from .mattn import Config, Context, DeviceError, InvalidShape, UnsupportedShape  # noqa: F401

__all__ = ["Config", "Context", "DeviceError", "InvalidShape", "UnsupportedShape", "mattn", "workloads"]
