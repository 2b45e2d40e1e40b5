"""ctypes front-end of the CPU oracle (``oracle/vkop_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, the smoke check and the
benchmark's CPU-baseline legs.  The product package never imports it.

All functions take and return numpy arrays.  16-bit inputs are passed as the
raw bit patterns (``uint16``) together with a dtype tag.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

F32, F16, BF16 = 0, 1, 2
SUM_F32_SEQUENTIAL, SUM_F64 = 0, 1
VALUE_PROBABILITY, VALUE_RAW = 0, 1

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path) or os.path.exists(_build.SRC) and os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            path = _build.build()
        _lib = C.CDLL(path)
        _lib.oracle_order_key.restype = C.c_uint32
        _lib.oracle_order_key.argtypes = [C.c_float]
    return _lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _as_storage(x: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F32:
        assert x.dtype == np.float32, x.dtype
    else:
        if x.dtype == np.float16 and dtype == F16:
            x = x.view(np.uint16)
        assert x.dtype == np.uint16, x.dtype
    return x


def dtype_of(x: np.ndarray, hint: int | None = None) -> int:
    if hint is not None:
        return hint
    if x.dtype == np.float32:
        return F32
    if x.dtype == np.float16:
        return F16
    raise ValueError("pass dtype= for uint16 bit patterns")


def softmax_topk(logits: np.ndarray, k: int, inv_temperature: float = 1.0, dtype: int | None = None,
                 value_kind: int = VALUE_PROBABILITY, sum_mode: int = SUM_F64, full_sort: bool = False):
    """Fused softmax + top-k of a 2-D array.  Returns (values f32 [rows,k], indices i64 [rows,k])."""
    dt = dtype_of(logits, dtype)
    x = _as_storage(logits, dt)
    assert x.ndim == 2
    rows, cols = x.shape
    stride = x.strides[0] // x.itemsize
    assert x.strides[1] == x.itemsize
    vals = np.empty((rows, k), np.float32)
    idx = np.empty((rows, k), np.int64)
    rc = lib().oracle_softmax_topk(_ptr(x), C.c_int(dt), C.c_int64(rows), C.c_int64(cols), C.c_int64(stride),
                                   C.c_int(k), C.c_float(inv_temperature), C.c_int(value_kind), C.c_int(sum_mode),
                                   C.c_int(int(full_sort)), _ptr(vals), _ptr(idx))
    if rc != 0:
        raise ValueError("oracle_softmax_topk: bad argument")
    return vals, idx


def softmax(x: np.ndarray, axis: int = -1, inv_temperature: float = 1.0, dtype: int | None = None,
            sum_mode: int = SUM_F64) -> np.ndarray:
    dt = dtype_of(x, dtype)
    xs = np.ascontiguousarray(_as_storage(x, dt))
    axis = axis % xs.ndim
    outer = int(np.prod(xs.shape[:axis], dtype=np.int64))
    inner = int(np.prod(xs.shape[axis + 1:], dtype=np.int64))
    out = np.empty(xs.shape, np.float32)
    rc = lib().oracle_softmax(_ptr(xs), C.c_int(dt), C.c_int64(outer), C.c_int64(xs.shape[axis]), C.c_int64(inner),
                              C.c_float(inv_temperature), C.c_int(sum_mode), _ptr(out))
    if rc != 0:
        raise ValueError("oracle_softmax: bad argument")
    return out


def topk(x: np.ndarray, k: int, axis: int = -1, largest: bool = True, sorted: bool = True, dtype: int | None = None):
    dt = dtype_of(x, dtype)
    xs = np.ascontiguousarray(_as_storage(x, dt))
    axis = axis % xs.ndim
    outer = int(np.prod(xs.shape[:axis], dtype=np.int64))
    inner = int(np.prod(xs.shape[axis + 1:], dtype=np.int64))
    oshape = list(xs.shape)
    oshape[axis] = k
    vals = np.empty(oshape, np.float32)
    idx = np.empty(oshape, np.int64)
    rc = lib().oracle_topk(_ptr(xs), C.c_int(dt), C.c_int64(outer), C.c_int64(xs.shape[axis]), C.c_int64(inner),
                           C.c_int(k), C.c_int(int(largest)), C.c_int(int(sorted)), _ptr(vals), _ptr(idx))
    if rc != 0:
        raise ValueError("oracle_topk: bad argument")
    return vals, idx


def shard_packet(shard: np.ndarray, k: int, index_offset: int, inv_temperature: float = 1.0, dtype: int | None = None):
    """Per-shard (m, s, keys, global indices, count) of every row."""
    dt = dtype_of(shard, dtype)
    x = _as_storage(shard, dt)
    rows, cols = x.shape
    stride = x.strides[0] // x.itemsize
    m = np.empty(rows, np.float32)
    s = np.empty(rows, np.float64)
    keys = np.empty((rows, k), np.uint32)
    idx = np.empty((rows, k), np.int64)
    cnt = np.empty(rows, np.int32)
    rc = lib().oracle_shard_packet(_ptr(x), C.c_int(dt), C.c_int64(rows), C.c_int64(cols), C.c_int64(stride),
                                   C.c_int64(index_offset), C.c_int(k), C.c_float(inv_temperature), _ptr(m), _ptr(s),
                                   _ptr(keys), _ptr(idx), _ptr(cnt))
    if rc != 0:
        raise ValueError("oracle_shard_packet: bad argument")
    return m, s, keys, idx, cnt


def merge_stats(m: np.ndarray, s: np.ndarray):
    m = np.ascontiguousarray(m, np.float32)
    s = np.ascontiguousarray(s, np.float64)
    mo = C.c_float()
    so = C.c_double()
    lib().oracle_merge_stats(_ptr(m), _ptr(s), C.c_int(m.shape[0]), C.byref(mo), C.byref(so))
    return mo.value, so.value


def sample_topk(values: np.ndarray, indices: np.ndarray, top_p: float, u: np.ndarray, dtype: int | None = None):
    """Sampling tail over the k survivors per row.  Returns (choice int32 [rows], token int64 [rows])."""
    dt = dtype_of(values, dtype)
    v = np.ascontiguousarray(_as_storage(values, dt))
    idx = np.ascontiguousarray(indices, np.int64)
    uu = np.ascontiguousarray(u, np.float32)
    rows, k = v.shape
    choice = np.empty(rows, np.int32)
    token = np.empty(rows, np.int64)
    rc = lib().oracle_sample_topk(_ptr(v), C.c_int(dt), _ptr(idx), C.c_int64(rows), C.c_int(k), C.c_float(top_p), _ptr(uu),
                                  _ptr(choice), _ptr(token))
    if rc != 0:
        raise ValueError("oracle_sample_topk: bad argument")
    return choice, token


def nms(boxes: np.ndarray, scores: np.ndarray, center_point_box: int = 0, max_output_boxes_per_class: int = 0,
        iou_threshold: float = 0.0, score_threshold: float = 0.0, pre_topk: int = 0, capacity_rows: int | None = None):
    """Returns (rows int32 [count,3], total count, per-(b,c) kept counts)."""
    boxes = np.ascontiguousarray(boxes, np.float32)
    scores = np.ascontiguousarray(scores, np.float32)
    B, N, four = boxes.shape
    assert four == 4
    Bs, Cn, Ns = scores.shape
    assert Bs == B and Ns == N
    cap = B * Cn * N if capacity_rows is None else capacity_rows
    rows = np.full((max(cap, 1), 3), -1, np.int32)
    total = C.c_int64()
    per = np.zeros(max(B * Cn, 1), np.int32)
    rc = lib().oracle_nms(_ptr(boxes), _ptr(scores), C.c_int(B), C.c_int(Cn), C.c_int(N), C.c_int(center_point_box),
                          C.c_int(max_output_boxes_per_class), C.c_float(iou_threshold), C.c_float(score_threshold),
                          C.c_int(pre_topk), _ptr(rows), C.c_int64(cap), C.byref(total), _ptr(per))
    if rc != 0:
        raise ValueError("oracle_nms: bad argument")
    n = min(total.value, cap)
    return rows[:n].copy(), total.value, per[:B * Cn].copy()


def ref_topk_bitonic(row: np.ndarray, k: int):
    """Emulation of the reference's multi-pass bitonic TopK on one fp32 row."""
    row = np.ascontiguousarray(row, np.float32)
    vals = np.empty(k, np.float32)
    idx = np.empty(k, np.int32)
    rc = lib().oracle_ref_topk_bitonic(_ptr(row), C.c_int(row.shape[0]), C.c_int(k), _ptr(vals), _ptr(idx))
    if rc != 0:
        raise ValueError("oracle_ref_topk_bitonic: bad argument (k must be < 256)")
    return vals, idx


def ref_softmax2_row(row: np.ndarray) -> np.ndarray:
    row = np.ascontiguousarray(row, np.float32)
    out = np.empty_like(row)
    lib().oracle_ref_softmax2_row(_ptr(row), C.c_int(row.shape[0]), _ptr(out))
    return out


def ref_nms_problem(boxes_n4: np.ndarray, scores_n: np.ndarray, center_point_box: int, max_output_boxes_per_class: int,
                    iou_threshold: float, score_threshold: float) -> np.ndarray:
    boxes_n4 = np.ascontiguousarray(boxes_n4, np.float32)
    scores_n = np.ascontiguousarray(scores_n, np.float32)
    kept = np.empty(1024, np.int32)
    lib().oracle_ref_nms_problem.restype = C.c_int
    n = lib().oracle_ref_nms_problem(_ptr(boxes_n4), _ptr(scores_n), C.c_int(scores_n.shape[0]),
                                     C.c_int(center_point_box), C.c_int(max_output_boxes_per_class),
                                     C.c_float(iou_threshold), C.c_float(score_threshold), _ptr(kept))
    return kept[:n].copy()


def ref_unfused_softmax_topk(logits: np.ndarray, k: int, inv_temperature: float = 1.0, dtype: int | None = None):
    """Emulation of the reference's UNFUSED order (ops/Softmax.hpp:61-141 followed by ops/Topk.hpp:95-217 on the
    softmax output): the probabilities are rounded to the pipeline's storage type first (fp32, or fp16 / bf16 bits),
    and TopK then selects on those rounded probabilities (value descending, lower index first among equal values),
    whereas the fused operator selects on the stored logits.  Distinct logits can round to equal probabilities, so
    the two orders may differ; this function is there to list where.  Returns (rounded probabilities f32 [rows,k],
    indices i64 [rows,k])."""
    dt = dtype_of(logits, dtype)
    x = _as_storage(logits, dt)
    p = softmax(x, -1, inv_temperature, dtype=dt, sum_mode=SUM_F32_SEQUENTIAL)
    if dt == F16:
        p = p.astype(np.float16).astype(np.float32)
    elif dt == BF16:
        b = p.view(np.uint32)
        b = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)  # round to nearest even
        p = b.view(np.float32)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    return np.take_along_axis(p, order, axis=1), order.astype(np.int64)


def to_oracle_array(x) -> np.ndarray:
    """CPU torch tensor -> numpy array in the oracle's storage convention (16-bit types as uint16 bits)."""
    import torch

    x = x.detach().cpu()
    if x.dtype == torch.float32:
        return x.numpy()
    return x.view(torch.int16).numpy().view(np.uint16)


def oracle_dtype(torch_dtype) -> int:
    """The oracle's dtype tag of a torch dtype."""
    import torch

    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[torch_dtype]


def order_key(x: float) -> int:
    return int(lib().oracle_order_key(C.c_float(x)))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(C.c_int(n))
