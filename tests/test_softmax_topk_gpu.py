"""GPU parity of the fused Softmax + TopK (C ABI) against the CPU oracle."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import oracle
from tests import util
from vkop_b200 import workloads

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c

    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return c


def test_reference_topk_cases(capi):
    """tests/TopkTest.cpp cases (seed 56): standalone TopK on the stored inputs, against the stored torch outputs."""
    g = np.load(os.path.join(GOLDEN, "topk_seed56.npz"))
    for n in range(5):
        k = int(g[f"case{n}_k"])
        x = torch.from_numpy(g[f"case{n}_f32_input"])
        v, i = capi.softmax_topk(x.cuda(), k, standalone_topk=True)
        assert np.array_equal(i.cpu().numpy(), g[f"case{n}_f32_indices"])
        assert np.array_equal(v.cpu().numpy(), g[f"case{n}_f32_values"])
        xh = torch.from_numpy(g[f"case{n}_f16_input"].view(np.float16))
        v, i = capi.softmax_topk(xh.cuda(), k, standalone_topk=True)
        # fp16 random data holds equal values; torch.topk's tie order is not canonical -> compare values bit-exactly
        # and indices with the oracle
        assert np.array_equal(v.cpu().numpy().view(np.uint16), g[f"case{n}_f16_values"])
        _, wi = oracle.topk(g[f"case{n}_f16_input"], k, dtype=oracle.F16)
        assert np.array_equal(i.cpu().numpy(), wi)


def test_classifier_head(capi):
    x = workloads.classifier_head()
    util.check_fused(x, 5, what="C1")


def test_batched_classifier_ties_int64(capi):
    x = workloads.batched_classifier()
    vals, idx = util.check_fused(x, 5, what="C2", index_dtype=capi.I64)
    assert idx.dtype == torch.int64
    # the quantised rows do hold ties inside the top 5 somewhere; the canonical order is (value desc, index asc)
    st = torch.sort(x, dim=1, stable=True, descending=True)[1][:, :5]
    assert torch.equal(idx.cpu(), st)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_llm_vocab(capi, dtype):
    x = workloads.llm_vocab(dtype=dtype)
    util.check_fused(x, workloads.LLM_K, workloads.LLM_INV_TEMPERATURE, what=f"C3 {dtype}")


def test_llm_vocab_deterministic(capi):
    x = workloads.llm_vocab().cuda()
    a = capi.softmax_topk(x, 50, 1.25)
    b = capi.softmax_topk(x, 50, 1.25)
    torch.cuda.synchronize()
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_sharded_vocab_shape_single_gpu(capi):
    x = workloads.sharded_vocab(rows=32)
    util.check_fused(x, 64, what="C5 rows[0:32] on one GPU")


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_exhaustive(capi, dtype):
    """Every n in 1..70 and every k in 1..n, on rows holding ties, signed zeros and infinities."""
    g = torch.Generator().manual_seed(11)
    for n in range(1, 71):
        x = torch.randn(6, n, generator=g)
        x[1] = torch.round(x[1] * 2) / 2          # heavy ties
        x[2] = 0.0
        x[2, ::2] = -0.0                          # signed zeros only
        x[3, ::3] = float("-inf")
        x[4] = 1.5                                # all equal
        if n > 2:
            x[5, 1] = float("inf") if n % 2 else 3.0
        x = x.to(dtype)
        for k in range(1, n + 1):
            if k > 128:
                break
            util.check_fused(x, k, what=f"n={n} k={k} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unaligned_rows(capi, dtype):
    """Row starts that are not 16-byte aligned (odd strides, offset base pointers)."""
    g = torch.Generator().manual_seed(12)
    for cols, stride, off in [(1000, 1001, 1), (777, 779, 3), (4099, 4101, 5), (20000, 20003, 2)]:
        buf = torch.randn(8 * stride + 16, generator=g).to(dtype)
        x_cpu = buf[off:off + 8 * stride].view(8, stride)[:, :cols]
        bg = buf.cuda()
        xg = bg[off:off + 8 * stride].view(8, stride)[:, :cols]
        vals, idx = capi.softmax_topk(xg, 9)
        wv, wi = util.oracle_softmax_topk(x_cpu.contiguous(), 9)
        util.assert_indices_equal(idx, wi, f"unaligned cols={cols}")
        util.assert_probs_close(vals, wv, dtype, f"unaligned cols={cols}")


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 8, 16, 33])
def test_forced_splits(capi, splits):
    g = torch.Generator().manual_seed(13)
    x = torch.randn(5, 16000, generator=g)
    x[0, :4000] = x[0, 4000:8000]  # duplicated values across chunks -> ties across packets
    util.check_fused(x, 50, 1.25, what=f"splits={splits}", splits=splits)


def test_few_rows_many_chunks(capi):
    g = torch.Generator().manual_seed(14)
    x = torch.randn(1, 300000, generator=g)
    util.check_fused(x, 64, what="1 x 300000")
    x = torch.randn(3, 1000003, generator=g).to(torch.bfloat16)
    util.check_fused(x, 17, what="3 x 1000003 bf16")


def test_fallback_paths(capi):
    """Inputs that defeat the threshold filter: all-equal rows, massive ties, NaN."""
    x = torch.zeros(4, 40000)
    x[1] = 2.0
    x[2, 777] = 3.0
    x[3] = torch.arange(40000) % 7
    util.check_fused(x, 50, what="all-equal / massive ties")
    for dt in (torch.float16, torch.bfloat16):
        util.check_fused(x.to(dt), 50, what=f"massive ties {dt}")
    # NaN ranks above +inf (torch ordering); the probabilities of such a row are NaN
    y = torch.randn(2, 5000, generator=torch.Generator().manual_seed(15))
    y[0, 1234] = float("nan")
    y[0, 99] = float("nan")
    y[1, 7] = float("inf")
    vals, idx = capi.softmax_topk(y.cuda(), 5)
    wv, wi = util.oracle_softmax_topk(y, 5)
    util.assert_indices_equal(idx, wi, "NaN rows")
    assert idx[0, 0].item() == 99 and idx[0, 1].item() == 1234
    assert torch.isnan(vals[0]).all()


def test_raw_value_kind_and_smallest(capi):
    g = torch.Generator().manual_seed(16)
    x = torch.randn(7, 3000, generator=g)
    x[0, 5] = -0.0
    x[0, 6] = 0.0
    xg = x.cuda()
    v, i = capi.softmax_topk(xg, 11, value_kind=capi.VALUE_RAW)
    wv, wi = oracle.topk(x.numpy(), 11)
    assert np.array_equal(i.cpu().numpy(), wi) and np.array_equal(v.cpu().numpy().view(np.uint32), wv.view(np.uint32))
    v, i = capi.softmax_topk(xg, 11, standalone_topk=True, largest=False)
    wv, wi = oracle.topk(x.numpy(), 11, largest=False)
    assert np.array_equal(i.cpu().numpy(), wi) and np.array_equal(v.cpu().numpy().view(np.uint32), wv.view(np.uint32))


def test_index_offset(capi):
    x = torch.randn(3, 2000, generator=torch.Generator().manual_seed(17))
    _, i0 = capi.softmax_topk(x.cuda(), 8)
    _, i1 = capi.softmax_topk(x.cuda(), 8, index_offset=123456, index_dtype=capi.I64)
    assert torch.equal(i0.long() + 123456, i1)


def test_partial_and_merge_single_device(capi):
    """Vocabulary sharding emulated on one GPU: packets of G column slices, merged."""
    x = workloads.sharded_vocab(rows=16, cols=64000)
    xg = x.cuda()
    k = 64
    for G in (1, 2, 4, 8):
        w = x.shape[1] // G
        packets = torch.stack([capi.softmax_topk_partial(xg[:, g * w:(g + 1) * w], k, g * w) for g in range(G)])
        vals, idx = capi.softmax_topk_merge(packets, x.shape[0], k, x.dtype)
        wv, wi = util.oracle_softmax_topk(x, k)
        util.assert_indices_equal(idx, wi, f"G={G}")
        util.assert_probs_close(vals, wv, x.dtype, f"G={G}")


def test_argument_errors(capi):
    x = torch.randn(2, 100).cuda()
    with pytest.raises(capi.VkopError) as e:
        capi.softmax_topk(x, 101)
    assert e.value.status == capi.INVALID_ARG
    with pytest.raises(capi.VkopError):
        capi.softmax_topk(x, 0)
    with pytest.raises(capi.VkopError):
        capi.softmax_topk(x, 5, inv_temperature=0.0)
    with pytest.raises(capi.VkopError):
        capi.softmax_topk(x, 5, inv_temperature=float("nan"))
    d = capi.make_desc(x, 5)
    import ctypes as C
    L = capi.lib()
    assert L.vkop_cuda_softmax_topk(C.byref(d), None, None, None, None, 0, None) == capi.INVALID_ARG
    assert L.vkop_cuda_softmax_topk(None, None, None, None, None, 0, None) == capi.INVALID_ARG
    # too small a workspace for a multi-chunk plan
    y = torch.randn(4, 200000).cuda()
    d = capi.make_desc(y, 50)
    need = capi.softmax_topk_workspace_bytes(d)
    assert need > 0
    v = torch.empty(4, 50).cuda()
    i = torch.empty(4, 50, dtype=torch.int32).cuda()
    small = torch.empty(16, dtype=torch.uint8).cuda()
    rc = L.vkop_cuda_softmax_topk(C.byref(d), y.data_ptr(), v.data_ptr(), i.data_ptr(), small.data_ptr(), 16, None)
    assert rc == capi.WORKSPACE_TOO_SMALL
    # zero rows is a valid no-op
    z = torch.empty(0, 100).cuda()
    capi.softmax_topk(z, 5)


# ---- streaming path (persistent CTAs, running threshold) ----

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_stream_llm_vocab(capi, dtype):
    x = workloads.llm_vocab(dtype=dtype)
    util.check_fused(x, workloads.LLM_K, workloads.LLM_INV_TEMPERATURE, what=f"stream C3 {dtype}", path=capi.PATH_STREAM)


def test_stream_is_the_automatic_choice_for_large_batches(capi):
    x = workloads.llm_vocab().cuda()
    a = capi.softmax_topk(x, 50, 1.25)
    b = capi.softmax_topk(x, 50, 1.25, path=capi.PATH_STREAM)
    c = capi.softmax_topk(x, 50, 1.25, path=capi.PATH_CHUNK)
    torch.cuda.synchronize()
    assert torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])
    assert torch.equal(a[1], c[1])


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_odd_shapes(capi, dtype):
    """CTA ranges that span several rows, unaligned row starts, rows shorter than a tile."""
    g = torch.Generator().manual_seed(51)
    for rows, cols, stride, off, k in [(300, 5000, 5000, 0, 9), (37, 20011, 20013, 3, 50), (5, 300007, 300007, 1, 64),
                                       (1000, 129, 131, 0, 4), (3, 1, 1, 0, 1), (2, 2049, 2049, 0, 128)]:
        buf = torch.randn(rows * stride + 16, generator=g).to(dtype)
        x_cpu = buf[off:off + rows * stride].view(rows, stride)[:, :cols]
        xg = buf.cuda()[off:off + rows * stride].view(rows, stride)[:, :cols]
        vals, idx = capi.softmax_topk(xg, k, 1.25, path=capi.PATH_STREAM)
        wv, wi = util.oracle_softmax_topk(x_cpu.contiguous(), k, 1.25)
        util.assert_indices_equal(idx, wi, f"stream {rows}x{cols} {dtype}")
        util.assert_probs_close(vals, wv, dtype, f"stream {rows}x{cols} {dtype}")


def test_stream_fallback_paths(capi):
    x = torch.zeros(6, 70000)
    x[1] = 2.0
    x[2, 777] = 3.0
    x[3] = (torch.arange(70000) % 7).float()
    x[4] = torch.arange(70000).float()           # ascending: the running threshold keeps rising
    x[5] = -torch.arange(70000).float()
    util.check_fused(x, 50, what="stream ties", path=capi.PATH_STREAM)
    y = torch.randn(3, 90000, generator=torch.Generator().manual_seed(52))
    y[0, 1234] = float("nan")
    y[0, 80000] = float("nan")
    y[2, 5] = float("-inf")
    vals, idx = capi.softmax_topk(y.cuda(), 5, path=capi.PATH_STREAM)
    wv, wi = util.oracle_softmax_topk(y, 5)
    util.assert_indices_equal(idx, wi, "stream NaN rows")
    assert torch.isnan(vals[0]).all() and not torch.isnan(vals[1:]).any()


def test_stream_back_to_back_with_input_ready(capi):
    """Overlapping launches (programmatic dependent launch) on one workspace and one output buffer."""
    xs = [workloads.llm_vocab(seed=60 + i).cuda() for i in range(3)]
    d = capi.make_desc(xs[0], 50, 1.25, flags=capi.FLAG_INPUT_READY)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
    ref = [capi.softmax_topk(x, 50, 1.25, path=capi.PATH_CHUNK) for x in xs]
    outs = [(torch.empty_like(ref[0][0]), torch.empty_like(ref[0][1])) for _ in xs]
    torch.cuda.synchronize()
    for rep in range(20):
        for x, o in zip(xs, outs):
            capi.softmax_topk(x, 50, 1.25, workspace=ws, out=o, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    for o, r in zip(outs, ref):
        assert torch.equal(o[1], r[1])
        assert torch.allclose(o[0], r[0], rtol=1e-5, atol=1e-7)
    # same buffer for consecutive launches: the last launch wins, nothing is torn
    o = outs[0]
    for rep in range(10):
        for x in xs:
            capi.softmax_topk(x, 50, 1.25, workspace=ws, out=o, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    assert torch.equal(o[1], ref[2][1])


@pytest.mark.parametrize("rows,cols,k,dtype", [(16, 128256, 50, torch.float32),   # four parts per row, scratch lists
                                               (5, 300007, 64, torch.float32),    # many parts, odd length
                                               (64, 70001, 8, torch.float16),     # whole rows, 16-bit
                                               (200, 40000, 32, torch.bfloat16),  # more rows than CTA pairs: CTAs cross rows
                                               (1, 1 << 20, 16, torch.float32)])  # one long row
def test_stream_overlapping_calls_in_every_launch_shape(capi, rows, cols, k, dtype):
    """Back-to-back calls that may overlap (the caller vouches for the logits), one workspace, one output
    buffer: every call's result must be intact when the next one is enqueued behind it."""
    g = torch.Generator().manual_seed(rows * 7 + k)
    xs = [torch.randn(rows, cols, generator=g).to(dtype) for _ in range(3)]
    xg = [x.cuda() for x in xs]
    want = [util.oracle_softmax_topk(x, k, 1.25) for x in xs]
    d = capi.make_desc(xg[0], k, 1.25, path=capi.PATH_STREAM, flags=capi.FLAG_INPUT_READY)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
    outs = [(torch.empty((rows, k), dtype=dtype, device="cuda"), torch.empty((rows, k), dtype=torch.int32, device="cuda"))
            for _ in xs]
    for rep in range(12):
        for x, o in zip(xg, outs):
            capi.softmax_topk(x, k, 1.25, workspace=ws, out=o, path=capi.PATH_STREAM, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    for o, (wv, wi) in zip(outs, want):
        util.assert_indices_equal(o[1], wi, f"overlapping {rows}x{cols}")
        util.assert_probs_close(o[0], wv, dtype, f"overlapping {rows}x{cols}")
    # one output buffer for all calls: the last call's result stands
    o = outs[0]
    for rep in range(6):
        for x in xg:
            capi.softmax_topk(x, k, 1.25, workspace=ws, out=o, path=capi.PATH_STREAM, flags=capi.FLAG_INPUT_READY)
    torch.cuda.synchronize()
    util.assert_indices_equal(o[1], want[2][1], f"overlapping, shared output {rows}x{cols}")


@pytest.mark.parametrize("dtype,index64,cols", [(torch.float32, False, 128256), (torch.float16, True, 70001)])
def test_overlapping_whole_row_calls_deliver_in_call_order(capi, dtype, index64, cols):
    """One CTA per row, several hundred calls in flight one behind the other on one workspace: a call whose
    predecessor has not finished a row leaves that row's result for the predecessor's CTA to deliver (the row's
    mailbox).  Two output buffers are written in turn from five inputs; a kernel enqueued right behind the last
    call (the copies below) must see, in either buffer, the result of the last call that wrote it."""
    rows, k, calls = 64, 50, 403
    g = torch.Generator().manual_seed(cols + k)
    xs = [(torch.randn(rows, cols, generator=g) * 2).to(dtype) for _ in range(5)]
    xg = [x.cuda() for x in xs]
    itype = capi.I64 if index64 else capi.I32
    d = capi.make_desc(xg[0], k, 1.25, itype, path=capi.PATH_STREAM, flags=capi.FLAG_INPUT_READY)
    ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
    outs = [(torch.zeros((rows, k), dtype=dtype, device="cuda"),
             torch.zeros((rows, k), dtype=torch.int64 if index64 else torch.int32, device="cuda")) for _ in range(2)]

    def enqueue():
        for i in range(calls):
            capi.softmax_topk(xg[i % 5], k, 1.25, index_dtype=itype, workspace=ws, out=outs[i % 2], path=capi.PATH_STREAM,
                              flags=capi.FLAG_INPUT_READY)

    enqueue()  # (from the host, slower than the device: little overlap)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()  # replayed, the calls run as deep as the GPU has room
    with torch.cuda.graph(graph):
        enqueue()
    for rep in range(4):
        for o in outs:
            o[0].zero_()
            o[1].zero_()
        graph.replay()
        seen = [(o[0].clone(), o[1].clone()) for o in outs]  # enqueued behind the last call, no synchronisation
        torch.cuda.synchronize()
        for b in range(2):
            last = max(i for i in range(calls) if i % 2 == b)
            wv, wi = util.oracle_softmax_topk(xs[last % 5], k, 1.25)
            util.assert_indices_equal(seen[b][1], wi, f"buffer {b}, round {rep}")
            util.assert_probs_close(seen[b][0], wv, dtype, f"buffer {b}, round {rep}")


@pytest.mark.parametrize("rows,cols,k,dtype", [(300, 9001, 5, torch.float32),      # just long enough, odd length
                                               (512, 32000, 64, torch.bfloat16),   # one GPU's slice of the sharded shape
                                               (592, 20000, 128, torch.float16),   # every light CTA slot taken, largest k
                                               (296, 70001, 50, torch.float32)])
def test_one_wave_of_whole_rows(capi, rows, cols, k, dtype):
    """Several hundred long rows: one light CTA per row, a single wave.  With and without VKOP_FLAG_INPUT_READY,
    from an unaligned pointer, with ties, NaN and infinities in some rows, raw values and the smallest."""
    g = torch.Generator().manual_seed(rows + cols + k)
    x = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
    x[1, : cols // 2] = x[1, cols // 2: 2 * (cols // 2)]  # every value twice: ties across the row
    x[2, 17] = float("nan")
    x[3, 5] = float("inf")
    x[4] = 1.5  # a constant row: the lowest indices win
    x[5, : cols - 3] = float("-inf")
    xg = x.cuda()
    wv, wi = util.oracle_softmax_topk(x, k, 1.25)
    for flags in (0, capi.FLAG_INPUT_READY):
        d = capi.make_desc(xg, k, 1.25, flags=flags)
        ws = capi.Workspace(capi.softmax_topk_workspace_bytes(d))
        out = (torch.empty((rows, k), dtype=dtype, device="cuda"), torch.empty((rows, k), dtype=torch.int32, device="cuda"))
        for rep in range(3):  # (calls with the flag overlap)
            capi.softmax_topk(xg, k, 1.25, workspace=ws, out=out, flags=flags)
        torch.cuda.synchronize()
        util.assert_indices_equal(out[1], wi, f"flags {flags}")
        util.assert_probs_close(out[0], wv, dtype, f"flags {flags}")
    # unaligned rows (a view that starts one element in), int64 indices
    xu = xg[:, 1:]
    wvu, wiu = util.oracle_softmax_topk(x[:, 1:].contiguous(), k, 1.0)
    v, i = capi.softmax_topk(xu, k, 1.0, index_dtype=capi.I64)
    torch.cuda.synchronize()
    util.assert_indices_equal(i, wiu, "unaligned")
    util.assert_probs_close(v, wvu, dtype, "unaligned")
    # standalone TopK, smallest
    kk = min(k, 17)
    v, i = capi.softmax_topk(xg, kk, standalone_topk=True, largest=False)
    torch.cuda.synchronize()
    wvs, wis = oracle.topk(util.to_oracle_array(x), kk, largest=False, dtype=util.ORACLE_DTYPE[dtype])
    assert np.array_equal(i.cpu().numpy(), wis)


def test_overlapping_calls_on_two_workspaces_in_turn(capi):
    """Calls with the flag on two workspaces (two shapes, two sets of outputs) enqueued in turn on one stream, with a
    call without the flag and a small chunk-path call thrown in: every kernel ends after the one before it, so
    the copies enqueued behind the last call see the final results of both."""
    g = torch.Generator().manual_seed(2024)
    xa = [torch.randn(64, 128256, generator=g) for _ in range(3)]
    xb = [torch.randn(96, 70001, generator=g).to(torch.float16) for _ in range(2)]
    xs = torch.randn(8, 1000, generator=g).cuda()
    ga, gb = [x.cuda() for x in xa], [x.cuda() for x in xb]
    F = capi.FLAG_INPUT_READY
    wsa = capi.Workspace(capi.softmax_topk_workspace_bytes(capi.make_desc(ga[0], 50, 1.25, flags=F)))
    wsb = capi.Workspace(capi.softmax_topk_workspace_bytes(capi.make_desc(gb[0], 20, 1.0, flags=F)))
    oa = (torch.zeros((64, 50), device="cuda"), torch.zeros((64, 50), dtype=torch.int32, device="cuda"))
    ob = (torch.zeros((96, 20), dtype=torch.float16, device="cuda"), torch.zeros((96, 20), dtype=torch.int32, device="cuda"))

    def enqueue():
        for i in range(60):
            capi.softmax_topk(ga[i % 3], 50, 1.25, workspace=wsa, out=oa, flags=F)
            capi.softmax_topk(gb[i % 2], 20, 1.0, workspace=wsb, out=ob, flags=F)
            if i % 16 == 5:
                capi.softmax_topk(xs, 5)  # chunk path, launched in the usual way

    enqueue()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue()
    wa = util.oracle_softmax_topk(xa[59 % 3], 50, 1.25)
    wb = util.oracle_softmax_topk(xb[59 % 2], 20, 1.0)
    for rep in range(3):
        oa[1].zero_()
        ob[1].zero_()
        graph.replay()
        seen = (oa[0].clone(), oa[1].clone(), ob[0].clone(), ob[1].clone())
        torch.cuda.synchronize()
        util.assert_indices_equal(seen[1], wa[1], f"workspace A, round {rep}")
        util.assert_probs_close(seen[0], wa[0], torch.float32, f"workspace A, round {rep}")
        util.assert_indices_equal(seen[3], wb[1], f"workspace B, round {rep}")
        util.assert_probs_close(seen[2], wb[0], torch.float16, f"workspace B, round {rep}")


def test_stream_raw_smallest_and_packets(capi):
    g = torch.Generator().manual_seed(53)
    x = torch.randn(40, 70001, generator=g)
    xg = x.cuda()
    v, i = capi.softmax_topk(xg, 11, standalone_topk=True, largest=False, path=capi.PATH_STREAM)
    wv, wi = oracle.topk(x.numpy(), 11, largest=False)
    assert np.array_equal(i.cpu().numpy(), wi) and np.array_equal(v.cpu().numpy().view(np.uint32), wv.view(np.uint32))
    # packets from the streaming path merge like any other
    xb = workloads.sharded_vocab(rows=24, cols=131072)
    xbg = xb.cuda()
    half = xb.shape[1] // 2
    pk = torch.stack([capi.softmax_topk_partial(xbg[:, :half], 64, 0, path=capi.PATH_STREAM),
                      capi.softmax_topk_partial(xbg[:, half:], 64, half, path=capi.PATH_STREAM)])
    vals, idx = capi.softmax_topk_merge(pk, 24, 64, xb.dtype)
    wv, wi = util.oracle_softmax_topk(xb, 64)
    util.assert_indices_equal(idx, wi, "stream packets")
    util.assert_probs_close(vals, wv, xb.dtype, "stream packets")
