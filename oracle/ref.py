"""ctypes front-end of ``oracle/_ref``: the reference's own CPU code for this path, compiled from its sources
by ``oracle/build_ref.py`` (TEST INFRASTRUCTURE ONLY; the product package never imports it).

``available()`` tells whether the libraries exist (they are built where the reference checkout is present
and travel with the repository snapshot from there)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_ref as _b

_lib = None
_lib_nms = None


def available(nms: bool = False) -> bool:
    _b.build(with_nms=nms)
    return os.path.exists(_b.LIB_NMS if nms else _b.LIB)


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("oracle/_ref is not built and there is no reference checkout to build it from")
        _lib = C.CDLL(_b.LIB)
    return _lib


def lib_nms():
    global _lib_nms
    if _lib_nms is None:
        if not available(nms=True):
            raise RuntimeError("oracle/_ref (NMS part) is not built and there is no reference checkout to build it from")
        import torch  # noqa: F401  (loads libtorch, which the library links)

        _lib_nms = C.CDLL(_b.LIB_NMS)
    return _lib_nms


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def function_top_k_predictions(x: np.ndarray, k: int, inv_temperature: float = 1.0):
    """core/function.cpp Function::get_top_k_predictions on every row of a float32 [rows, cols] array (rows in
    parallel).  Returns (indices int32 [rows, k], probabilities float32 [rows, k])."""
    assert x.dtype == np.float32 and x.ndim == 2 and x.strides[1] == 4
    rows, cols = x.shape
    idx = np.empty((rows, k), np.int32)
    prob = np.empty((rows, k), np.float32)
    rc = lib().ref_function_top_k_predictions(_p(x), C.c_int64(rows), C.c_int64(cols), C.c_int64(x.strides[0] // 4),
                                              C.c_float(inv_temperature), C.c_int(k), _p(idx), _p(prob))
    if rc != 0:
        raise ValueError("ref_function_top_k_predictions: bad argument")
    return idx, prob


def softmax_nd(x: np.ndarray, axis: int) -> np.ndarray:
    """tests/SoftmaxTest.cpp softmax_nd on a float32 array of rank <= 4 (leading dimensions of 1 are added)."""
    assert x.dtype == np.float32 and x.ndim <= 4
    x = np.ascontiguousarray(x)
    shape = (1,) * (4 - x.ndim) + x.shape
    axis = axis % x.ndim + (4 - x.ndim)
    out = np.empty(shape, np.float32)
    rc = lib().ref_softmax_nd(_p(x), _p(out), *[C.c_int(s) for s in shape], C.c_int(axis))
    if rc != 0:
        raise ValueError("ref_softmax_nd: bad argument")
    return out.reshape(x.shape)


def topk_rows(x: np.ndarray, k: int):
    """tests/TopkTest.cpp get_top_k_predictions.  Returns (column indices int32 [rows, k], values [rows, k])."""
    assert x.dtype == np.float32 and x.ndim == 2
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    idx = np.empty((rows, k), np.int32)
    val = np.empty((rows, k), np.float32)
    rc = lib().ref_topk_rows(_p(x), C.c_int(rows), C.c_int(cols), C.c_int(k), _p(idx), _p(val))
    if rc != 0:
        raise ValueError("ref_topk_rows: bad argument")
    return idx - (np.arange(rows, dtype=np.int32) * cols)[:, None], val


def nms_expected(boxes: np.ndarray, scores: np.ndarray, iou_threshold: float, score_threshold: float) -> np.ndarray:
    """tests/NmsTest.cpp NmsTest::compute_expected_nms: rows (batch, class, box) int32 [n, 3]."""
    assert boxes.dtype == np.float32 and scores.dtype == np.float32
    boxes, scores = np.ascontiguousarray(boxes), np.ascontiguousarray(scores)
    B, N, four = boxes.shape
    assert four == 4 and scores.shape[0] == B and scores.shape[2] == N
    Cn = scores.shape[1]
    cap = B * Cn * N
    rows = np.empty((cap, 3), np.int32)
    n = lib_nms().ref_nms_expected(_p(boxes), _p(scores), C.c_int(B), C.c_int(Cn), C.c_int(N), C.c_float(iou_threshold),
                                   C.c_float(score_threshold), _p(rows), C.c_int(cap))
    if n < 0:
        raise ValueError("ref_nms_expected failed")
    return rows[:n].copy()


def set_num_threads(n: int) -> None:
    """Threads of the row loop in function_top_k_predictions (OpenMP)."""
    import ctypes.util

    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        C.CDLL(ctypes.util.find_library("gomp") or "libgomp.so.1").omp_set_num_threads(C.c_int(n))
    except OSError:
        pass
