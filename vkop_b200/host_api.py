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
           "vkop_host_model_describe", "vkop_host_model_run",
           "vkop_host_sharded_create", "vkop_host_sharded_destroy", "vkop_host_sharded_ipc_handle", "vkop_host_sharded_connect",
           "vkop_host_sharded_connect_local", "vkop_host_sharded_begin", "vkop_host_sharded_finish", "vkop_host_sharded_run",
           "vkop_host_sharded_timed_out")

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
        L.vkop_host_sharded_create.restype = C.c_void_p
        L.vkop_host_sharded_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int,
                                               C.c_float, C.c_uint]
        L.vkop_host_sharded_destroy.argtypes = [C.c_void_p]
        L.vkop_host_sharded_ipc_handle.argtypes = [C.c_void_p, C.c_void_p]
        L.vkop_host_sharded_connect.argtypes = [C.c_void_p, C.c_void_p]
        L.vkop_host_sharded_connect_local.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        L.vkop_host_sharded_begin.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.vkop_host_sharded_finish.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.vkop_host_sharded_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.vkop_host_sharded_timed_out.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
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


class ShardedRank:
    """One rank of the vocabulary-sharded fused Softmax + TopK, owned by the C++ operator ops::SoftmaxTopkSharded
    (scratch, receive buffer, IPC mapping, step numbers, the partial -> push -> wait -> merge chain).  The caller
    moves the 64-byte handles between the ranks: `handle()` on every rank, `connect(all handles in rank order)`,
    a barrier, then `run` (or `begin` on every rank followed by `finish`).  Ranks of one process use
    `connect_local(list of ShardedRank)`.  Pointers are raw device addresses; `stream` is a cudaStream_t."""

    def __init__(self, device: int, rank: int, world: int, rows: int, cols_local: int, col_offset: int, k: int, dtype: int,
                 index_dtype: int = 0, inv_temperature: float = 1.0, max_polls: int = 0):
        self.rank, self.world = rank, world
        self._h = lib().vkop_host_sharded_create(device, rank, world, rows, cols_local, col_offset, k, dtype, index_dtype,
                                                 float(inv_temperature), max_polls)
        if not self._h:
            raise RuntimeError("vkop_host_sharded_create: " + lib().vkop_host_last_error().decode())

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what}: status {rc}: " + lib().vkop_host_last_error().decode())

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        self._check(lib().vkop_host_sharded_ipc_handle(self._h, buf), "vkop_host_sharded_ipc_handle")
        return buf.raw

    def connect(self, handles) -> None:
        blob = b"".join(handles)
        assert len(blob) == 64 * self.world
        self._check(lib().vkop_host_sharded_connect(self._h, blob), "vkop_host_sharded_connect")

    def connect_local(self, ranks) -> None:
        arr = (C.c_void_p * self.world)(*[r._h for r in ranks])
        self._check(lib().vkop_host_sharded_connect_local(self._h, arr), "vkop_host_sharded_connect_local")

    def begin(self, logits_ptr: int, stream: int = 0) -> None:
        self._check(lib().vkop_host_sharded_begin(self._h, logits_ptr, stream), "vkop_host_sharded_begin")

    def finish(self, values_ptr: int, indices_ptr: int, stream: int = 0) -> None:
        self._check(lib().vkop_host_sharded_finish(self._h, values_ptr, indices_ptr, stream), "vkop_host_sharded_finish")

    def run(self, logits_ptr: int, values_ptr: int, indices_ptr: int, stream: int = 0) -> None:
        self._check(lib().vkop_host_sharded_run(self._h, logits_ptr, values_ptr, indices_ptr, stream), "vkop_host_sharded_run")

    def timed_out(self) -> bool:
        t = C.c_int(0)
        self._check(lib().vkop_host_sharded_timed_out(self._h, C.byref(t)), "vkop_host_sharded_timed_out")
        return bool(t.value)

    def close(self) -> None:
        if self._h:
            lib().vkop_host_sharded_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
