"""CPU tests: the oracle against the golden fixtures and torch-CPU, the reference-emulation variants, and the
host-side logic that needs no GPU."""
from __future__ import annotations

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import oracle
from tests import util
from vkop_b200 import workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def test_oracle_topk_matches_reference_test_vectors():
    g = np.load(os.path.join(GOLDEN, "topk_seed56.npz"))
    for n in range(5):
        k = int(g[f"case{n}_k"])
        v, i = oracle.topk(g[f"case{n}_f32_input"], k)
        assert np.array_equal(i, g[f"case{n}_f32_indices"])
        assert np.array_equal(v, g[f"case{n}_f32_values"])
        xh = g[f"case{n}_f16_input"]
        v, i = oracle.topk(xh, k, dtype=oracle.F16)
        want = g[f"case{n}_f16_values"].view(np.float16).astype(np.float32)
        assert np.array_equal(v, want)  # values are tie-order independent
        st = torch.sort(torch.from_numpy(xh.view(np.float16)).float(), dim=1, stable=True, descending=True)[1][:, :k]
        assert np.array_equal(i, st.numpy())


def test_oracle_softmax_matches_reference_test_vectors():
    g = np.load(os.path.join(GOLDEN, "softmax_seed42.npz"))
    for n in range(6):
        axis = int(g[f"case{n}_axis"])
        x = g[f"case{n}_f32_input"]
        y = oracle.softmax(x, axis)
        want = g[f"case{n}_f32_output"]
        assert np.all(np.abs(y - want) <= 1e-6 + 1e-5 * np.abs(want))
        y_seq = oracle.softmax(x, axis, sum_mode=oracle.SUM_F32_SEQUENTIAL)
        assert np.all(np.abs(y_seq - want) <= 1e-6 + 1e-5 * np.abs(want))
        xh = g[f"case{n}_f16_input"]
        yh = oracle.softmax(xh, axis, dtype=oracle.F16)
        wanth = g[f"case{n}_f16_output"].view(np.float16).astype(np.float32)
        assert np.all(np.abs(yh - wanth) <= 6e-8 + 2e-3 * np.abs(wanth))


def test_oracle_nms_matches_reference_test_expectations():
    g = np.load(os.path.join(GOLDEN, "nms_cases.npz"))
    for n in range(3):
        max_per_class, iou_thr, score_thr = g[f"case{n}_params"]
        rows, total, per = oracle.nms(g[f"case{n}_boxes"], g[f"case{n}_scores"], iou_threshold=float(iou_thr),
                                      score_threshold=float(score_thr))
        want = g[f"case{n}_expected"]
        assert total == want.shape[0] and np.array_equal(rows, want)
        if max_per_class > 0:
            rows2, total2, per2 = oracle.nms(g[f"case{n}_boxes"], g[f"case{n}_scores"], iou_threshold=float(iou_thr),
                                             score_threshold=float(score_thr),
                                             max_output_boxes_per_class=int(max_per_class))
            assert np.all(per2 == np.minimum(per, int(max_per_class)))
            # per (batch, class) the capped result is a prefix of the uncapped one
            off = off2 = 0
            for p_full, p_cap in zip(per, per2):
                assert np.array_equal(rows[off:off + p_cap], rows2[off2:off2 + p_cap])
                off += p_full
                off2 += p_cap


def test_oracle_fused_against_torch_on_workloads():
    for x, k, inv_t in [(workloads.classifier_head(), 5, 1.0), (workloads.batched_classifier(), 5, 1.0),
                        (workloads.llm_vocab(rows=4), 50, 1.25)]:
        v, i = oracle.softmax_topk(x.numpy(), k, inv_t)
        st = torch.sort(x, dim=1, stable=True, descending=True)[1][:, :k]
        assert np.array_equal(i, st.numpy())
        p = torch.softmax(x.double() * float(np.float32(inv_t)), -1).gather(1, st).numpy()
        assert np.all(np.abs(v - p) <= 1e-6 + 1e-5 * np.abs(p))
        # the reference's own CPU statement (sequential fp32 sum, full sort) agrees on indices and, loosely, on values
        v2, i2 = oracle.softmax_topk(x.numpy(), k, inv_t, sum_mode=oracle.SUM_F32_SEQUENTIAL, full_sort=True)
        assert np.array_equal(i2, i)
        assert np.all(np.abs(v2 - p) <= 1e-6 + 1e-4 * np.abs(p))


def test_oracle_ties_zeros_nan_order():
    x = np.array([[1.0, -0.0, 0.0, 1.0, np.inf, np.nan, -np.inf, 0.0]], np.float32)
    _, i = oracle.topk(x, 8)
    assert i[0].tolist() == [5, 4, 0, 3, 1, 2, 7, 6]
    _, i = oracle.topk(x, 3, largest=False)
    assert i[0].tolist() == [6, 1, 2]
    assert oracle.order_key(-0.0) == oracle.order_key(0.0)


def test_vocab_sharding_merge_equals_unsharded():
    x = workloads.sharded_vocab(rows=6, cols=8000)
    xa = util.to_oracle_array(x)
    k = 64
    wv, wi = oracle.softmax_topk(xa, k, dtype=oracle.BF16)
    from vkop_b200.sharded import split_even
    for G in (1, 2, 3, 4, 8):
        packets = []
        for g in range(G):
            lo, hi = split_even(x.shape[1], G, g)
            packets.append(oracle.shard_packet(np.ascontiguousarray(xa[:, lo:hi]), k, lo, dtype=oracle.BF16))
        v, i = util.merge_packets_reference(packets, k, xa, oracle.BF16)
        assert np.array_equal(i, wi)
        assert np.all(np.abs(v - wv) <= 1e-6 + 1e-5 * np.abs(wv))


def test_split_even_covers_everything():
    from vkop_b200.sharded import split_even
    for n in (0, 1, 7, 64, 256000, 128256):
        for w in (1, 2, 3, 4, 8):
            parts = [split_even(n, w, r) for r in range(w)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[r][1] == parts[r + 1][0] for r in range(w - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1


def test_reference_emulation_differences():
    """Where the reference shaders depart from the canonical contract (kept as documentation of the differences)."""
    g = torch.Generator().manual_seed(5)
    # tie-free data: the multi-pass bitonic TopK agrees with the canonical order
    x = torch.randn(2000, generator=g).numpy()
    v, i = oracle.ref_topk_bitonic(x, 7)
    cv, ci = oracle.topk(x[None], 7)
    assert np.array_equal(i, ci[0]) and np.array_equal(v, cv[0])
    # tie-heavy data: same values, but equal values come out in network order, not lowest index first
    differ = 0
    for t in range(20):
        xt = (torch.randint(0, 8, (600,), generator=g).float() / 4).numpy()
        v, i = oracle.ref_topk_bitonic(xt, 7)
        cv, ci = oracle.topk(xt[None], 7)
        assert np.array_equal(v, cv[0])
        differ += int(not np.array_equal(i, ci[0]))
    assert differ > 0
    # softmax2.comp's summation tree agrees with the canonical softmax within the contract tolerance
    row = torch.randn(1000, generator=g).numpy()
    a, b = oracle.ref_softmax2_row(row), oracle.softmax(row[None])[0]
    assert np.all(np.abs(a - b) <= 1e-6 + 1e-5 * np.abs(b))
    # nms.comp on a problem with fewer than 1024 candidates and distinct scores: same kept boxes
    xy = torch.rand(300, 2, generator=g) * 20
    boxes = torch.cat([xy, xy + torch.rand(300, 2, generator=g) * 6 + 0.5], -1).numpy()
    scores = torch.rand(300, generator=g).numpy()
    kept = oracle.ref_nms_problem(boxes, scores, 0, 0, 0.4, 0.1)
    rows, _, _ = oracle.nms(boxes[None], scores[None, None], iou_threshold=0.4, score_threshold=0.1)
    assert np.array_equal(kept, rows[:, 2])
    # ... and with more than 1024 candidates the shader only considers the first 1024 by index
    xy = torch.rand(3000, 2, generator=g) * 200
    boxes = torch.cat([xy, xy + torch.rand(3000, 2, generator=g) * 6 + 0.5], -1).numpy()
    scores = torch.rand(3000, generator=g).numpy()
    kept = oracle.ref_nms_problem(boxes, scores, 0, 0, 0.4, 0.1)
    rows, _, _ = oracle.nms(boxes[None], scores[None, None], iou_threshold=0.4, score_threshold=0.1)
    assert kept.max() < 1200 and rows[:, 2].max() > 1200


def test_c_abi_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "vkop_cuda.h")).read()
    declared = sorted(set(re.findall(r"\b(vkop_cuda_\w+)\s*\(", header)))
    assert len(declared) >= 12
    from vkop_b200 import capi
    lib = ctypes.CDLL(capi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(capi.EXPORTS) == [d for d in declared if d in capi.EXPORTS]
    missing_binding = [d for d in declared if d not in capi.EXPORTS]
    assert not missing_binding, missing_binding
    # calls that need no device
    assert lib.vkop_cuda_version() == 100
    lib.vkop_cuda_status_string.restype = ctypes.c_char_p
    assert lib.vkop_cuda_status_string(-1) == b"VKOP_INVALID_ARG"
    lib.vkop_cuda_packet_bytes.restype = ctypes.c_size_t
    assert lib.vkop_cuda_packet_bytes(64) == (4 + 128) * 4


def test_host_library_exports_its_entry_points():
    """libvkop_host.so (the C++ operator API and its flat C entry points) loads without a device and exports
    what the Python front end binds, the vocabulary-sharded operator included."""
    from vkop_b200 import host_api
    lib = ctypes.CDLL(host_api.HOST_LIB_PATH)
    for name in host_api.EXPORTS:
        assert hasattr(lib, name), name
    assert any(n.startswith("vkop_host_sharded_") for n in host_api.EXPORTS)


def test_workspace_planning_needs_no_device():
    from vkop_b200 import capi
    d = capi.SoftmaxTopkDesc(rows=64, cols=128256, row_stride=128256, dtype=capi.F32, k=50, index_dtype=capi.I32,
                             value_kind=0, inv_temperature=1.25, largest=1, path=0, splits=0, index_offset=0)
    assert capi.softmax_topk_workspace_bytes(d) > 0
    d.k = 0
    n = ctypes.c_size_t()
    assert capi.lib().vkop_cuda_softmax_topk_workspace(ctypes.byref(d), ctypes.byref(n)) == capi.INVALID_ARG
    d.k = 1024  # served by the radix path
    assert capi.softmax_topk_workspace_bytes(d) > 0
    d.k = 5000
    assert capi.lib().vkop_cuda_softmax_topk_workspace(ctypes.byref(d), ctypes.byref(n)) == capi.INVALID_ARG


def test_planner_serves_every_shape_and_flag_without_a_device():
    """The planners are host code: sweep shapes, element types, k, paths and the overlap flag, and check that
    every supported combination gets a finite scratch size and every refusal is a status, not a crash."""
    from vkop_b200 import capi
    n = ctypes.c_size_t()
    fn = capi.lib().vkop_cuda_softmax_topk_workspace
    served = 0
    for rows in (1, 2, 5, 16, 64, 148, 149, 300, 512, 4096, 100000):
        for cols in (1, 7, 1000, 16384, 32000, 128256, 256000, 300007, 1 << 20, 1 << 24):
            if rows * cols > (1 << 34):
                continue
            for dtype in (capi.F32, capi.F16, capi.BF16):
                for k in (1, 5, 50, 64, 128, 300, 1024):
                    if k > cols:
                        continue
                    for path in (capi.PATH_AUTO, capi.PATH_CHUNK, capi.PATH_STREAM, capi.PATH_RADIX):
                        for flags in (0, capi.FLAG_INPUT_READY):
                            d = capi.SoftmaxTopkDesc(rows=rows, cols=cols, row_stride=cols, dtype=dtype, k=k,
                                                     index_dtype=capi.I32, value_kind=0, inv_temperature=1.0, largest=1,
                                                     path=path, splits=0, index_offset=0, flags=flags, reserved=0)
                            rc = fn(ctypes.byref(d), ctypes.byref(n))
                            assert rc in (capi.OK, capi.UNSUPPORTED), (rows, cols, dtype, k, path, flags, rc)
                            if rc == capi.OK:
                                served += 1
                                assert 0 <= n.value < (64 << 30), (rows, cols, k, path, n.value)
                            if path == capi.PATH_AUTO:
                                assert rc == capi.OK, ("the automatic choice must serve", rows, cols, dtype, k, flags)
    assert served > 5000


def test_workspace_holds_the_rows_mailboxes():
    """Shapes that run one CTA per row keep, per row, an order word, a ticket counter and a mailbox of 16 entries
    (two addresses, k values, k indices, each block rounded up to 16 bytes): the planned scratch size must cover
    them, whatever the alignment of the logits turns out to be at the call."""
    from vkop_b200 import capi

    def up16(n):
        return (n + 15) // 16 * 16

    for rows, cols, flags in ((64, 128256, capi.FLAG_INPUT_READY), (148, 70001, capi.FLAG_INPUT_READY), (512, 256000, 0),
                              (296, 9001, capi.FLAG_INPUT_READY), (592, 20000, 0)):
        for dtype, esz in ((capi.F32, 4), (capi.BF16, 2)):
            for k in (1, 50, 128):
                for itype, isz in ((capi.I32, 4), (capi.I64, 8)):
                    d = capi.SoftmaxTopkDesc(rows=rows, cols=cols, row_stride=cols, dtype=dtype, k=k, index_dtype=itype,
                                             value_kind=0, inv_temperature=1.0, largest=1, path=capi.PATH_STREAM, splits=0,
                                             index_offset=0, flags=flags, reserved=0)
                    need = rows * 16 * (16 + up16(k * esz) + up16(k * isz)) + 2 * rows * 4
                    assert capi.softmax_topk_workspace_bytes(d) >= need, (rows, cols, dtype, k, itype)


def test_oracle_sampling_known_answers():
    v = np.array([[0.5, 0.3, 0.1, 0.05]], np.float32)
    ids = np.array([[7, 3, 9, 1]])
    pick = lambda top_p, u: tuple(int(a[0]) for a in oracle.sample_topk(v, ids, top_p, np.array([u], np.float32)))
    # all four kept (sum 0.95): prefix sums 0.5 / 0.8 / 0.9 / 0.95 against u * 0.95
    assert pick(1.0, 0.0) == (0, 7) and pick(1.0, 0.51) == (0, 7)
    assert pick(1.0, 0.85) == (2, 9) and pick(1.0, 0.99) == (3, 1)
    # top_p 0.8: 0.76 is reached by the first two; draws stay inside them
    assert pick(0.8, 0.85) == (1, 3) and pick(0.8, 0.99) == (1, 3) and pick(0.8, 0.1) == (0, 7)
    # a tiny nucleus is the best candidate alone
    assert pick(0.01, 0.999) == (0, 7)
    with pytest.raises(ValueError):
        oracle.sample_topk(v, ids, 0.0, np.array([0.5], np.float32))


def test_product_has_no_cpu_path():
    from vkop_b200 import capi
    x = torch.randn(2, 100)
    try:
        capi.softmax_topk(x, 5)
    except RuntimeError as e:
        assert "CUDA" in str(e)
    else:
        raise AssertionError("a CPU tensor must be rejected")
    src = open(os.path.join(ROOT, "vkop_b200", "capi.py")).read() + open(os.path.join(ROOT, "vkop_b200", "sharded.py")).read()
    assert "import oracle" not in src and "from oracle" not in src


def test_unfused_order_emulation_against_the_contract():
    """The reference runs Softmax, rounds the probabilities to the pipeline's type, then TopK on those; the fused
    operator selects on the stored logits.  On every benchmark configuration the two orders give the same indices
    (the rows where they differ are counted and must be none); a crafted fp16 row whose two runner-up
    probabilities round to the same subnormal shows what a difference looks like."""
    cases = [("C1", workloads.classifier_head(), 5, 1.0), ("C2", workloads.batched_classifier(), 5, 1.0),
             ("C3 f32", workloads.llm_vocab(rows=16), 50, 1.25),
             ("C3 f16", workloads.llm_vocab(dtype=torch.float16), 50, 1.25),
             ("C5 bf16", workloads.sharded_vocab(rows=8), 64, 1.0)]
    for name, x, k, inv_t in cases:
        xa, dt = util.to_oracle_array(x), util.ORACLE_DTYPE[x.dtype]
        _, i = oracle.softmax_topk(xa, k, inv_t, dtype=dt)
        _, pi = oracle.ref_unfused_softmax_topk(xa, k, inv_t, dtype=dt)
        differing = int((i != pi).any(axis=1).sum())
        assert differing == 0, f"{name}: {differing} rows where the unfused order differs"
    x = torch.full((1, 64), -30.0, dtype=torch.float16)
    x[0, 0] = 10.0
    x[0, 5] = -5.004   # fp16 neighbours: distinct logits ...
    x[0, 9] = -5.0     # ... whose probabilities (3e-7) round to one fp16 subnormal
    xa = util.to_oracle_array(x)
    assert xa[0, 5] != xa[0, 9]
    _, i = oracle.softmax_topk(xa, 3, dtype=oracle.F16)
    pv, pi = oracle.ref_unfused_softmax_topk(xa, 3, dtype=oracle.F16)
    assert list(i[0]) == [0, 9, 5]            # the contract: larger logit first
    assert pv[0, 1] == pv[0, 2] and list(pi[0]) == [0, 5, 9]   # the unfused order: equal probabilities, lower index first
