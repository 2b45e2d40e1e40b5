"""GPU parity of TopK along any axis and of the unsorted output order (C ABI vkop_cuda_topk_axis) against the oracle.

The reference accepts the attributes "axis" (0 .. 2) and "sorted" (ops/Topk.hpp:62-79, 98-103); its own test only
runs the last axis, sorted (tests/TopkTest.cpp:91-125), so the expectation here is the oracle's TopK on the same view:
value order with lower index first among equal values, and ascending index order when sorted = 0."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from tests.util import to_oracle_array

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c

    assert torch.cuda.is_available()
    return c


def check(capi, x: torch.Tensor, k: int, axis: int, largest: bool, sorted_: bool, index_dtype=None):
    index_dtype = capi.I32 if index_dtype is None else index_dtype
    vals, idx = capi.topk_axis(x.cuda(), k, axis=axis, largest=largest, sorted=sorted_, index_dtype=index_dtype)
    torch.cuda.synchronize()
    wv, wi = oracle.topk(to_oracle_array(x), k, axis=axis, largest=largest, sorted=sorted_, dtype=oracle.oracle_dtype(x.dtype))
    assert tuple(vals.shape) == wv.shape
    assert np.array_equal(idx.cpu().numpy().astype(np.int64), wi), (tuple(x.shape), k, axis, largest, sorted_)
    got = vals.float().cpu().numpy()
    assert np.array_equal(got.view(np.uint32), wv.view(np.uint32)) or np.array_equal(np.nan_to_num(got), np.nan_to_num(wv))
    assert idx.dtype == (torch.int64 if index_dtype == capi.I64 else torch.int32)


def rounded(shape, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.round(torch.randn(*shape, generator=g) * 16) / 16).to(dtype)  # many equal values


@pytest.mark.parametrize("sorted_", [True, False])
@pytest.mark.parametrize("largest", [True, False])
def test_reference_shapes_on_every_axis(capi, largest, sorted_):
    """[3, 2000] along axis 0 and 1 (tests/TopkTest.cpp:93-99 shapes), 3-D tensors along each axis."""
    check(capi, rounded((3, 2000), 1), 2, 0, largest, sorted_)
    check(capi, rounded((3, 2000), 2), 3, 0, largest, sorted_)
    check(capi, rounded((3, 2000), 3), 7, 1, largest, sorted_)
    check(capi, rounded((1, 600), 4), 7, -1, largest, sorted_)
    for axis in (0, 1, 2, -2):
        check(capi, rounded((4, 50, 33), 5 + axis), 4 if axis == 0 else 5, axis, largest, sorted_)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_dtypes_index_types_and_odd_extents(capi, dtype):
    check(capi, rounded((2, 300, 5), 11, dtype), 9, 1, True, False)
    check(capi, rounded((7, 129, 31), 12, dtype), 33, 1, True, True, capi.I64)
    check(capi, rounded((5, 64, 40), 13, dtype), 64, 1, False, False, capi.I64)  # k = the whole axis
    check(capi, rounded((1, 1, 17), 14, dtype), 1, 1, True, False)
    check(capi, rounded((33, 2), 15, dtype), 1, 0, True, True)
    check(capi, rounded((2, 5000, 3), 16, dtype), 300, 1, True, False)


def test_long_axis_with_inner_extent(capi):
    """An axis long enough for the streaming selection ([40000, 64] along axis 0: 64 rows of 40000 after the turn)."""
    g = torch.Generator().manual_seed(17)
    x = torch.randn(40000, 64, generator=g)
    check(capi, x, 50, 0, True, True)
    check(capi, x, 50, 0, True, False)
    check(capi, x, 1024, 0, False, False)


def test_unsorted_last_axis_large_k(capi):
    g = torch.Generator().manual_seed(18)
    x = torch.randn(16, 30000, generator=g)
    check(capi, x, 4096, -1, True, False)
    check(capi, x, 1000, -1, False, False, capi.I64)


def test_argument_errors(capi):
    import ctypes as C

    L = capi.lib()
    n = C.c_size_t()
    d = capi.TopkAxisDesc(outer=2, axis_len=10, inner=3, dtype=0, k=11, index_dtype=0, largest=1, sorted=1, path=0)
    assert L.vkop_cuda_topk_axis_workspace(C.byref(d), C.byref(n)) == capi.INVALID_ARG  # k beyond the axis
    d.k = 3
    d.index_dtype = 5
    assert L.vkop_cuda_topk_axis_workspace(C.byref(d), C.byref(n)) == capi.INVALID_ARG
    d.index_dtype = 0
    assert L.vkop_cuda_topk_axis_workspace(C.byref(d), C.byref(n)) == capi.OK and n.value > 0
    assert L.vkop_cuda_topk_axis(C.byref(d), None, None, None, None, 0, None) == capi.INVALID_ARG
    x = torch.zeros(2, 10, 3, device="cuda")
    v = torch.zeros(2, 3, 3, device="cuda")
    i = torch.zeros(2, 3, 3, dtype=torch.int32, device="cuda")
    assert L.vkop_cuda_topk_axis(C.byref(d), x.data_ptr(), v.data_ptr(), i.data_ptr(), None, 0, None) == capi.WORKSPACE_TOO_SMALL
    d.outer = 0  # nothing to do
    assert L.vkop_cuda_topk_axis(C.byref(d), None, None, None, None, 0, None) == capi.OK
