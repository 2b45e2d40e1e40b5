"""ctypes front-end of libvkop_host.so, the C++ mirror of the reference's operator / Runtime API.

A HostPipeline is what the reference's benchmark program builds
(benchmark/main.cpp:85-118): a Runtime whose model output is a [rows, cols]
logits tensor, with Softmax and TopK registered as post-processing, then
Run() and ReadResult().  It takes HOST buffers: the logits are copied to the
device, the operators run through the C ABI, the k values and indices of every
row come back to host memory.  There is no CPU fallback: without the built
library, or without a CUDA device, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(HERE, "libvkop_host.so")
EXPORTS = ("vkop_host_pipeline_create", "vkop_host_pipeline_run", "vkop_host_pipeline_destroy", "vkop_host_last_error",
           "vkop_host_model_describe", "vkop_host_model_run")

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(HOST_LIB_PATH):
            raise RuntimeError(f"{HOST_LIB_PATH} is missing: build it with `python -m vkop_b200.build`")
        L = C.CDLL(HOST_LIB_PATH)
        L.vkop_host_pipeline_create.restype = C.c_void_p
        L.vkop_host_pipeline_create.argtypes = [C.c_int] * 5 + [C.c_float, C.c_int]
        L.vkop_host_pipeline_run.restype = C.c_int
        L.vkop_host_pipeline_run.argtypes = [C.c_void_p] * 5
        L.vkop_host_pipeline_destroy.argtypes = [C.c_void_p]
        L.vkop_host_last_error.restype = C.c_char_p
        _lib = L
    return _lib


class HostPipeline:
    """Softmax -> TopK registered on a logits tensor, run from host buffers.

    dtype: 0 f32, 1 f16, 2 bf16 (the C ABI's vkop_dtype).  temperature divides the
    logits as the reference's sampling path does; fuse=False runs the two
    registered operators one after the other instead of the fused one.
    """

    def __init__(self, device: int, rows: int, cols: int, dtype: int, k: int, temperature: float = 1.0, fuse: bool = True):
        self.rows, self.cols, self.k, self.dtype = rows, cols, k, dtype
        self._h = lib().vkop_host_pipeline_create(device, rows, cols, dtype, k, float(temperature), 1 if fuse else 0)
        if not self._h:
            raise RuntimeError("vkop_host_pipeline_create: " + lib().vkop_host_last_error().decode())

    def run_ptr(self, logits_ptr: int, values_ptr: int, indices_ptr: int) -> float:
        """Raw host addresses in, device milliseconds of Runtime::Run() out."""
        ms = C.c_double()
        rc = lib().vkop_host_pipeline_run(self._h, logits_ptr, values_ptr, indices_ptr, C.addressof(ms))
        if rc != 0:
            raise RuntimeError(f"vkop_host_pipeline_run: status {rc}: " + lib().vkop_host_last_error().decode())
        return ms.value

    def run(self, logits, values, indices) -> float:
        """numpy arrays (C-contiguous, host): logits [rows, cols], values [rows, k], indices int32 [rows, k]."""
        assert logits.flags["C_CONTIGUOUS"] and values.flags["C_CONTIGUOUS"] and indices.flags["C_CONTIGUOUS"]
        assert logits.shape == (self.rows, self.cols) and values.shape == (self.rows, self.k) and indices.shape == (self.rows, self.k)
        return self.run_ptr(logits.ctypes.data, values.ctypes.data, indices.ctypes.data)

    def close(self):
        if self._h:
            lib().vkop_host_pipeline_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
