"""The entry point that takes no workspace and allocates nothing (vkop_cuda_softmax_topk_static).

Collected last on purpose: its scratch array is shared by every call of the process, so this file
checks that it behaves whatever ran before it, and also when it runs alone.
"""
from __future__ import annotations

import pytest
import torch

from vkop_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c
    return c


def _same(a, b):
    return torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])


def test_two_calls_in_a_row_match_the_workspace_entry_point(capi):
    x1 = workloads.llm_vocab(seed=7, rows=16).cuda()
    x2 = workloads.llm_vocab(seed=8, rows=16).cuda()
    want1 = capi.softmax_topk(x1, 50, 1.25, path=capi.PATH_CHUNK)
    want2 = capi.softmax_topk(x2, 50, 1.25, path=capi.PATH_CHUNK)
    got1 = capi.softmax_topk_static(x1, 50, 1.25)
    got2 = capi.softmax_topk_static(x2, 50, 1.25)   # same descriptor: the array is reused as it was left
    torch.cuda.synchronize()
    assert _same(got1, want1)
    assert _same(got2, want2)
    # and against the CPU oracle (indices bit for bit, probabilities within the fp32 tolerance)
    from tests import util

    for x, got in ((x1, got1), (x2, got2)):
        wv, wi = util.oracle_softmax_topk(x.cpu(), 50, 1.25)
        util.assert_indices_equal(got[1], wi, "static entry point")
        util.assert_probs_close(got[0], wv, torch.float32, "static entry point")


def test_descriptor_change_clears_what_it_must(capi):
    # different shapes lay their counters out differently in the shared array
    for rows, cols, k in [(3, 300007, 64), (256, 1000, 5), (16, 128256, 50), (1, 70001, 7)]:
        g = torch.Generator().manual_seed(rows * 31 + k)
        x = torch.randn(rows, cols, generator=g).cuda()
        want = capi.softmax_topk(x, k, path=capi.PATH_CHUNK)
        got = capi.softmax_topk_static(x, k)
        again = capi.softmax_topk_static(x, k)
        torch.cuda.synchronize()
        assert _same(got, want), (rows, cols, k)
        assert _same(again, want), (rows, cols, k)


def test_shapes_alternate_on_the_shared_array(capi):
    """Calls with different launch shapes lay their counters out differently in the one array; every call
    clears its own first, so they may alternate freely."""
    x = workloads.llm_vocab(seed=9, rows=16).cuda()
    y = torch.randn(3, 300007, generator=torch.Generator().manual_seed(10)).cuda()
    wx = capi.softmax_topk(x, 50, 1.25, path=capi.PATH_CHUNK)
    wy = capi.softmax_topk(y, 64, path=capi.PATH_CHUNK)
    for _ in range(3):
        gx = capi.softmax_topk_static(x, 50, 1.25)
        gy = capi.softmax_topk_static(y, 64)
        torch.cuda.synchronize()
        assert _same(gx, wx) and _same(gy, wy)


def test_limits_are_reported(capi):
    import ctypes as C

    assert capi.static_scratch_bytes() == 4 << 20
    x = torch.randn(4, 4096).cuda()
    v = torch.empty(4, 5, device="cuda")
    i = torch.empty(4, 5, dtype=torch.int32, device="cuda")
    fn = capi.lib().vkop_cuda_softmax_topk_static
    desc = capi.make_desc(x, 5, 1.0, path=capi.PATH_STREAM)
    # VKOP_UNSUPPORTED: only the chunk kernel works in the built-in array
    assert fn(C.byref(desc), x.data_ptr(), v.data_ptr(), i.data_ptr(), 0) == -2
    # VKOP_WORKSPACE_TOO_SMALL, before anything is launched: 2000 long rows in 8 chunks each need 66 MB of scratch
    big = capi.make_desc(x, 5, 1.0)
    big.rows, big.cols, big.row_stride, big.k, big.splits = 2000, 128256, 128256, 50, 8
    assert fn(C.byref(big), x.data_ptr(), v.data_ptr(), i.data_ptr(), 0) == -3
    # and the array still serves the next call
    want = capi.softmax_topk(x, 5, path=capi.PATH_CHUNK)
    got = capi.softmax_topk_static(x, 5)
    torch.cuda.synchronize()
    assert _same(got, want)
