"""GPU parity of the bulk-copy streaming kernel (VKOP_PATH_BULK) against the CPU oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from tests import util
from vkop_b200 import workloads

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return c


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_bulk_llm_vocab(capi, dtype):
    """The headline shape, 64 x 128256, against the oracle (indices bit-exact, probabilities within tolerance)."""
    x = workloads.llm_vocab(dtype=dtype)
    util.check_fused(x, workloads.LLM_K, workloads.LLM_INV_TEMPERATURE, what=f"bulk C3 {dtype}", path=capi.PATH_BULK)


@pytest.mark.parametrize("parts", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
def test_bulk_parts_per_row(capi, parts, dtype):
    """Every row is cut into `parts` streaming CTAs (desc.splits names the number); ragged row ends, ties
    across the parts of a row, k up to 128."""
    g = torch.Generator().manual_seed(76 + parts)
    epv = 4 if dtype == torch.float32 else 8
    for rows, cols, k in [(5, 70001, 50), (33, 131072 + 8, 128), (64, 128256, 1)]:
        if (cols + epv - 1) // epv // parts < 2048:
            continue
        stride = (cols + epv - 1) // epv * epv
        buf = torch.randn(rows * stride, generator=g).to(dtype)
        x_cpu = buf.view(rows, stride)[:, :cols]
        x_cpu[0, : cols // 2] = x_cpu[0, cols - cols // 2:]  # every value of row 0 twice, in different parts
        xg = buf.cuda().view(rows, stride)[:, :cols]
        vals, idx = capi.softmax_topk(xg, k, 1.25, path=capi.PATH_BULK, splits=parts)
        wv, wi = util.oracle_softmax_topk(x_cpu.contiguous(), k, 1.25)
        util.assert_indices_equal(idx, wi, f"{parts} parts: {rows}x{cols} {dtype}")
        util.assert_probs_close(vals, wv, dtype, f"{parts} parts: {rows}x{cols} {dtype}")


def test_bulk_agrees_with_the_other_paths(capi):
    x = workloads.llm_vocab().cuda()
    a = capi.softmax_topk(x, 50, 1.25)
    b = capi.softmax_topk(x, 50, 1.25, path=capi.PATH_BULK)
    c = capi.softmax_topk(x, 50, 1.25, path=capi.PATH_CHUNK)
    torch.cuda.synchronize()
    assert torch.equal(a[1], b[1]) and torch.equal(a[1], c[1])
    assert torch.allclose(a[0], b[0], rtol=1e-5, atol=1e-7)


def test_bulk_vocab_sharded_shape_all_rows(capi):
    """512 x 256000 bf16, k = 64: the full row count of the vocabulary-sharded configuration on one GPU."""
    x = workloads.sharded_vocab()
    util.check_fused(x, 64, what="bulk C5 512 rows", path=capi.PATH_BULK)


@pytest.mark.parametrize("dtype", DTYPES)
def test_bulk_odd_shapes(capi, dtype):
    """Ranges that span several rows, ragged row ends inside padded strides, short last tiles."""
    g = torch.Generator().manual_seed(71)
    epv = 4 if dtype == torch.float32 else 8
    for rows, cols, pad, k in [(300, 20000, 0, 9), (37, 40011, 5, 50), (7, 300007, 1, 64), (150, 16385, 7, 128),
                               (2, 70001, 3, 1), (1000, 16640, 0, 33)]:
        stride = (cols + pad + epv - 1) // epv * epv
        buf = torch.randn(rows * stride, generator=g).to(dtype)
        x_cpu = buf.view(rows, stride)[:, :cols]
        xg = buf.cuda().view(rows, stride)[:, :cols]
        try:
            vals, idx = capi.softmax_topk(xg, k, 1.25, path=capi.PATH_BULK)
        except capi.VkopError as e:
            assert e.status == capi.UNSUPPORTED  # a shape the bulk kernel leaves to the other paths
            vals, idx = capi.softmax_topk(xg, k, 1.25)
        wv, wi = util.oracle_softmax_topk(x_cpu.contiguous(), k, 1.25)
        util.assert_indices_equal(idx, wi, f"bulk {rows}x{cols} {dtype}")
        util.assert_probs_close(vals, wv, dtype, f"bulk {rows}x{cols} {dtype}")


def test_bulk_fallback_paths(capi):
    """Inputs that defeat the bound: all-equal rows, massive ties, monotone rows, NaN, infinities."""
    x = torch.zeros(8, 70000)
    x[1] = 2.0
    x[2, 777] = 3.0
    x[3] = (torch.arange(70000) % 7).float()
    x[4] = torch.arange(70000).float()
    x[5] = -torch.arange(70000).float()
    x[6] = float("-inf")
    x[6, 69999] = 1.0
    x[7] = float("-inf")
    util.check_fused(x, 50, what="bulk ties", path=capi.PATH_BULK)
    for dt in (torch.float16, torch.bfloat16):
        util.check_fused(x.to(dt), 50, what=f"bulk ties {dt}", path=capi.PATH_BULK)
    y = torch.randn(4, 90000, generator=torch.Generator().manual_seed(72))
    y[0, 1234] = float("nan")
    y[0, 80000] = float("nan")
    y[2, 5] = float("-inf")
    y[3, 77] = float("inf")
    vals, idx = capi.softmax_topk(y.cuda(), 5, path=capi.PATH_BULK)
    wv, wi = util.oracle_softmax_topk(y, 5)
    util.assert_indices_equal(idx, wi, "bulk NaN rows")
    util.assert_probs_close(vals, wv, torch.float32, "bulk NaN rows")
    assert torch.isnan(vals[0]).all() and not torch.isnan(vals[1:3]).any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", ["bulk", "stream", "chunk", "radix"])
def test_sparse_nan_without_a_sum(capi, dtype, path):
    """Standalone TopK and raw values carry no exp-sum that would show a NaN: NaN still ranks above +inf
    on every path, wherever it sits (alone in its thread's share of the row, far below the bound)."""
    pth = {"bulk": capi.PATH_BULK, "stream": capi.PATH_STREAM, "chunk": capi.PATH_CHUNK, "radix": capi.PATH_RADIX}[path]
    g = torch.Generator().manual_seed(73)
    x = torch.randn(6, 66000, generator=g)
    x[0, 12345] = float("nan")
    x[1, 0] = float("nan")
    x[1, 65999] = float("nan")
    x[2, 40000:40003] = float("nan")
    x[4, 5] = float("inf")
    x[4, 50000] = float("nan")
    x = x.to(dtype)
    xa = util.to_oracle_array(x)
    xg = x.cuda()
    for largest in (True, False):
        v, i = capi.softmax_topk(xg, 7, standalone_topk=True, largest=largest, path=pth)
        wv, wi = oracle.topk(xa, 7, largest=largest, dtype=util.ORACLE_DTYPE[dtype])
        util.assert_indices_equal(i, wi, f"NaN topk {path} {dtype} largest={largest}")
        got = v.float().cpu().numpy()
        assert ((got == wv) | (np.isnan(got) & np.isnan(wv))).all()
    v, i = capi.softmax_topk(xg, 7, value_kind=capi.VALUE_RAW, path=pth)
    _, wi = oracle.topk(xa, 7, dtype=util.ORACLE_DTYPE[dtype])
    util.assert_indices_equal(i, wi, f"NaN raw {path} {dtype}")


def test_bulk_raw_smallest_and_packets(capi):
    g = torch.Generator().manual_seed(74)
    x = torch.randn(40, 70004, generator=g)
    xg = x.cuda()
    v, i = capi.softmax_topk(xg, 11, standalone_topk=True, largest=False, path=capi.PATH_BULK)
    wv, wi = oracle.topk(x.numpy(), 11, largest=False)
    assert np.array_equal(i.cpu().numpy(), wi) and np.array_equal(v.cpu().numpy().view(np.uint32), wv.view(np.uint32))
    xb = workloads.sharded_vocab(rows=24, cols=131072)
    xbg = xb.cuda()
    half = xb.shape[1] // 2
    pk = torch.stack([capi.softmax_topk_partial(xbg[:, :half], 64, 0, path=capi.PATH_BULK),
                      capi.softmax_topk_partial(xbg[:, half:], 64, half, path=capi.PATH_BULK)])
    vals, idx = capi.softmax_topk_merge(pk, 24, 64, xb.dtype)
    wv, wi = util.oracle_softmax_topk(xb, 64)
    util.assert_indices_equal(idx, wi, "bulk packets")
    util.assert_probs_close(vals, wv, xb.dtype, "bulk packets")


@pytest.mark.parametrize("rows,cols,k,dtype", [(64, 128256, 50, torch.float32),   # the headline launch shape
                                               (16, 128256, 50, torch.float32),
                                               (200, 40000, 32, torch.bfloat16),  # CTAs cross rows, whole rows inside
                                               (512, 32000, 64, torch.bfloat16)])  # one GPU's slice of the sharded shape
def test_bulk_overlapping_calls(capi, rows, cols, k, dtype):
    """Back-to-back calls that may overlap (VKOP_FLAG_INPUT_READY), one workspace: every call's result is
    intact, against the oracle; with one output buffer for all calls the last call's result stands."""
    g = torch.Generator().manual_seed(rows * 7 + k)
    xs = [torch.randn(rows, cols, generator=g).to(dtype) for _ in range(3)]
    xg = [x.cuda() for x in xs]
    want = [util.oracle_softmax_topk(x, k, 1.25) for x in xs]
    d = capi.make_desc(xg[0], k, 1.25, path=capi.PATH_BULK, flags=capi.FLAG_INPUT_READY)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
    outs = [(torch.empty((rows, k), dtype=dtype, device="cuda"), torch.empty((rows, k), dtype=torch.int32, device="cuda"))
            for _ in xs]
    for rep in range(12):
        for x, o in zip(xg, outs):
            capi.softmax_topk(x, k, 1.25, workspace=ws, out=o, path=capi.PATH_BULK, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    for o, (wv, wi) in zip(outs, want):
        util.assert_indices_equal(o[1], wi, f"overlapping {rows}x{cols}")
        util.assert_probs_close(o[0], wv, dtype, f"overlapping {rows}x{cols}")
    o = outs[0]
    for rep in range(6):
        for x in xg:
            capi.softmax_topk(x, k, 1.25, workspace=ws, out=o, path=capi.PATH_BULK, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    util.assert_indices_equal(o[1], want[2][1], f"overlapping, shared output {rows}x{cols}")


def test_aligned_and_unaligned_pointers_share_a_workspace(capi):
    """The same descriptor with a 16-byte aligned and an unaligned logits pointer gets two different launch
    plans of the streaming kernel (another grid); the calls may alternate on one workspace, overlapping, with
    one output buffer."""
    g = torch.Generator().manual_seed(75)
    rows, cols, k = 48, 66000, 20
    base = torch.randn(rows * cols + 8, generator=g)
    xa_cpu = base[:rows * cols].view(rows, cols)
    xu_cpu = base[1:1 + rows * cols].view(rows, cols)
    bg = base.cuda()
    xa, xu = bg[:rows * cols].view(rows, cols), bg[1:1 + rows * cols].view(rows, cols)
    wa, wu = util.oracle_softmax_topk(xa_cpu.contiguous(), k), util.oracle_softmax_topk(xu_cpu.contiguous(), k)
    d = capi.make_desc(xa, k, flags=capi.FLAG_INPUT_READY)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
    o = (torch.empty((rows, k), device="cuda"), torch.empty((rows, k), dtype=torch.int32, device="cuda"))
    for rep in range(10):
        capi.softmax_topk(xa, k, workspace=ws, out=o, flags=capi.FLAG_INPUT_READY)
        capi.softmax_topk(xu, k, workspace=ws, out=o, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    util.assert_indices_equal(o[1], wu[1], "aligned then unaligned")
    capi.softmax_topk(xa, k, workspace=ws, out=o, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    util.assert_indices_equal(o[1], wa[1], "unaligned then aligned")
    util.assert_probs_close(o[0], wa[0], torch.float32, "unaligned then aligned")


@pytest.mark.parametrize("path_name", ["AUTO", "BULK"])
def test_many_overlapping_calls_keep_their_pace(capi, path_name):
    """Forty thousand overlapping calls replayed from a CUDA graph: every call numbers itself on the device from a
    counter its predecessor advances.  A call that read that counter too early shared its predecessor's number and
    sat out a bounded wait of a second; no replay may take anywhere near that, and the last result is right."""
    path = getattr(capi, "PATH_" + path_name)
    rows, cols, k = 64, 128256, 50
    g = torch.Generator().manual_seed(91)
    xs = [torch.randn(rows, cols, generator=g) for _ in range(4)]
    xg = [x.cuda() for x in xs]
    d = capi.make_desc(xg[0], k, 1.25, path=path, flags=capi.FLAG_INPUT_READY)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
    o = (torch.empty((rows, k), device="cuda"), torch.empty((rows, k), dtype=torch.int32, device="cuda"))
    for x in xg:
        capi.softmax_topk(x, k, 1.25, workspace=ws, out=o, path=path, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(256):
            capi.softmax_topk(xg[i % 4], k, 1.25, workspace=ws, out=o, path=path, flags=capi.FLAG_INPUT_READY)
    times = []
    for rep in range(160):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    assert times[-1] < 100.0 and times[-1] < 20 * times[len(times) // 2], (times[len(times) // 2], times[-5:])
    wv, wi = util.oracle_softmax_topk(xs[3], k, 1.25)
    util.assert_indices_equal(o[1], wi, "last of many overlapping calls")
    util.assert_probs_close(o[0], wv, torch.float32, "last of many overlapping calls")
