"""zeninfer_b200 -- B200 (sm_100a) backend for ZenInfer's block-quantised GEMV/GEMM path.

The product is the shared library ``lib/libzen_cuda.so`` (hand-written CUDA kernels behind the
C-ABI of ``include/zen_cuda.h``).  This package is the thin harness around it: ``backend`` binds
the C-ABI with ctypes and mirrors the reference's ``zen::quant`` call shapes, ``blocks`` packs and
decodes the GGUF block formats, ``shard`` plans row sharding across GPUs.

There is no CPU implementation here.  Every compute call raises if the library or a B200 is missing.
"""
from . import blocks  # noqa: F401
from .backend import Backend, BackendError, load_library  # noqa: F401

__all__ = ["Backend", "BackendError", "load_library", "blocks"]
