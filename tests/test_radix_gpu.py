"""GPU parity of the radix-select path (large k, long rows) against the CPU oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from tests import util
from vkop_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c

    assert torch.cuda.is_available()
    return c


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k", [1, 50, 300, 1024])
def test_radix_forced(capi, dtype, k):
    g = torch.Generator().manual_seed(31)
    x = torch.randn(5, 50021, generator=g)
    x[1] = torch.round(x[1] * 4) / 4  # heavy ties: the index digits decide
    x[2] = 0.25                        # one value: pure index selection
    x[3, 100:50000:7] = float("-inf")
    x = x.to(dtype)
    util.check_fused(x, k, 1.25, what=f"radix k={k} {dtype}", path=capi.PATH_RADIX)


def test_radix_small_rows(capi):
    g = torch.Generator().manual_seed(32)
    for n in (1, 2, 7, 33, 1000):
        x = torch.randn(3, n, generator=g)
        for k in sorted({1, n // 2 or 1, n}):
            util.check_fused(x, k, what=f"radix n={n} k={k}", path=capi.PATH_RADIX)


def test_auto_picks_radix_for_large_k(capi):
    g = torch.Generator().manual_seed(33)
    x = torch.randn(2, 8400, generator=g)
    util.check_fused(x, 300, what="k=300 auto")
    x = torch.randn(1, 700000, generator=g)
    util.check_fused(x, 1024, what="k=1024 auto")


def test_radix_unaligned_and_raw(capi):
    g = torch.Generator().manual_seed(34)
    buf = torch.randn(3 * 9001 + 8, generator=g)
    x_cpu = buf[1:1 + 3 * 9001].view(3, 9001)[:, :8999]
    xg = buf.cuda()[1:1 + 3 * 9001].view(3, 9001)[:, :8999]
    v, i = capi.softmax_topk(xg, 200, value_kind=capi.VALUE_RAW, path=capi.PATH_RADIX, index_dtype=capi.I64)
    wv, wi = oracle.topk(x_cpu.contiguous().numpy(), 200)
    assert np.array_equal(i.cpu().numpy(), wi)
    assert np.array_equal(v.cpu().numpy().view(np.uint32), wv.view(np.uint32))
    v, i = capi.softmax_topk(xg, 200, standalone_topk=True, largest=False, path=capi.PATH_RADIX)
    wv, wi = oracle.topk(x_cpu.contiguous().numpy(), 200, largest=False)
    assert np.array_equal(i.cpu().numpy(), wi)


def test_long_row_16m(capi):
    """One fp32 row of 16,777,216 elements, k = 1024."""
    x = workloads.long_row()
    util.check_fused(x, 1024, what="16Mi row k=1024")
    # same call twice on one workspace: scratch state must be left ready
    xg = x.cuda()
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(capi.make_desc(xg, 1024)))
    a = capi.softmax_topk(xg, 1024, workspace=ws)
    b = capi.softmax_topk(xg, 1024, workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])
