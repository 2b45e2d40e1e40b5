"""vkop_b200: sm_100a CUDA implementation of vkop's GPU post-processing path
(Softmax + TopK fused, NMS) behind a C ABI (``include/vkop_cuda.h``).

``vkop_b200.capi`` is a thin ctypes binding of that C ABI for the test and
benchmark harness; device memory and streams come from torch.  There is no CPU
path: loading fails if the CUDA library has not been built.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
