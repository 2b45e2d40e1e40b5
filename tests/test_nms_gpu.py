"""GPU parity of NMS (C ABI) against the CPU oracle and the stored reference-test expectations."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import oracle
from vkop_b200 import workloads

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c

    assert torch.cuda.is_available()
    return c


def run_both(capi, boxes, scores, **kw):
    rows, count = capi.nms(boxes.cuda(), scores.cuda(), **kw)
    torch.cuda.synchronize()
    n = int(count.item())
    want_rows, want_total, _ = oracle.nms(boxes.numpy(), scores.numpy(), **kw)
    assert n == want_total, (n, want_total)
    got = rows[:min(n, rows.shape[0])].cpu().numpy()
    assert np.array_equal(got, want_rows[:got.shape[0]])
    return got


def test_reference_nms_cases(capi):
    """tests/NmsTest.cpp:181-185 shapes and thresholds; expectation = the test's own greedy NMS (stored)."""
    g = np.load(os.path.join(GOLDEN, "nms_cases.npz"))
    for n in range(3):
        boxes, scores = torch.from_numpy(g[f"case{n}_boxes"]), torch.from_numpy(g[f"case{n}_scores"])
        max_per_class, iou_thr, score_thr = g[f"case{n}_params"]
        got = run_both(capi, boxes, scores, iou_threshold=float(iou_thr), score_threshold=float(score_thr))
        assert np.array_equal(got, g[f"case{n}_expected"])
        if max_per_class > 0:
            run_both(capi, boxes, scores, iou_threshold=float(iou_thr), score_threshold=float(score_thr),
                     max_output_boxes_per_class=int(max_per_class))


def test_yolo_detect_subset(capi):
    boxes, scores = workloads.yolo_detect(batch=2, classes=12)
    got = run_both(capi, boxes, scores, **workloads.YOLO_PARAMS)
    assert got.shape[0] > 0


def test_yolo_detect_full(capi):
    boxes, scores = workloads.yolo_detect()
    run_both(capi, boxes, scores, **workloads.YOLO_PARAMS)


def test_small_and_edge(capi):
    g = torch.Generator().manual_seed(41)
    for B, C, N in [(1, 1, 1), (2, 3, 5), (1, 2, 33), (3, 1, 257), (1, 1, 1000)]:
        xy = torch.rand(B, N, 2, generator=g) * 10
        wh = torch.rand(B, N, 2, generator=g) * 4 + 0.1
        boxes = torch.cat([xy, xy + wh], -1)
        scores = torch.rand(B, C, N, generator=g)
        scores[..., ::5] = scores[..., 1::5][..., :scores[..., ::5].shape[-1]] if N > 5 else scores[..., ::5]  # tied scores
        for kw in [dict(iou_threshold=0.5, score_threshold=0.1),
                   dict(iou_threshold=0.0, score_threshold=0.0),
                   dict(iou_threshold=0.3, score_threshold=0.5, max_output_boxes_per_class=3),
                   dict(iou_threshold=0.45, score_threshold=0.2, pre_topk=7, max_output_boxes_per_class=5),
                   dict(iou_threshold=1.0, score_threshold=0.0),
                   dict(iou_threshold=0.5, score_threshold=2.0)]:
            run_both(capi, boxes, scores, **kw)


def test_center_point_and_degenerate_boxes(capi):
    g = torch.Generator().manual_seed(42)
    N = 400
    boxes = torch.cat([torch.rand(1, N, 2, generator=g) * 50, torch.rand(1, N, 2, generator=g) * 20], -1)
    boxes[0, ::7, 2:] = 0.0          # zero-area boxes
    boxes[0, 5] = boxes[0, 6]        # identical boxes
    scores = torch.rand(1, 4, N, generator=g)
    scores[0, :, 5] = scores[0, :, 6]
    run_both(capi, boxes, scores, center_point_box=1, iou_threshold=0.4, score_threshold=0.05)


def test_large_candidate_sets(capi):
    """Problems beyond the bit-mask sweep (iterative sweep) and beyond the sort buffer (radix pre-selection)."""
    g = torch.Generator().manual_seed(43)
    N = 3000
    xy = torch.rand(1, N, 2, generator=g) * 300
    wh = torch.rand(1, N, 2, generator=g) * 30 + 1
    boxes = torch.cat([xy, xy + wh], -1)
    scores = torch.rand(1, 2, N, generator=g)
    run_both(capi, boxes, scores, iou_threshold=0.5, score_threshold=0.05)          # ~2850 candidates, no pre-selection
    run_both(capi, boxes, scores, iou_threshold=0.5, score_threshold=0.05, pre_topk=200)  # overflow of the 1024 sort buffer
    run_both(capi, boxes, scores, iou_threshold=0.5, score_threshold=0.05, pre_topk=1500, max_output_boxes_per_class=100)


def test_iou_next_to_the_threshold(capi):
    """Integer boxes give IoUs that are exact ratios (1/3, 1/2, 3/5 ...); with the threshold on such a ratio, one
    float above and one below, the test that avoids the division has to hand over to the exact one."""
    boxes = []
    for x in range(12):
        for w in (2, 3, 4, 6):
            boxes.append([x, 0.0, x + w, 1.0])
            boxes.append([x, 0.0, x + w, 2.0])
    boxes = torch.tensor(boxes, dtype=torch.float32)[None]
    N = boxes.shape[1]
    g = torch.Generator().manual_seed(44)
    scores = torch.rand(1, 3, N, generator=g) * 0.9 + 0.05
    for ratio in (1 / 3, 0.5, 0.6, 0.25, 2 / 3, 0.2, 0.75):
        t = np.float32(ratio)
        for thr in (t, np.nextafter(t, np.float32(1)), np.nextafter(t, np.float32(0))):
            run_both(capi, boxes, scores, iou_threshold=float(thr), score_threshold=0.0)


def test_areas_and_thresholds_outside_the_quick_range(capi):
    """Huge and tiny boxes (areas beyond 1e28 / below 1e-28), thresholds of 0, below 0 and tiny, boxes with NaN
    or infinite coordinates: all of these take the exact IoU."""
    g = torch.Generator().manual_seed(45)
    N = 200
    xy = torch.rand(1, N, 2, generator=g) * 10
    wh = torch.rand(1, N, 2, generator=g) * 6 + 0.5
    base = torch.cat([xy, xy + wh], -1)
    scores = torch.rand(1, 2, N, generator=g)
    for scale in (1e16, 1e-16, 1e19, 1e-19):
        run_both(capi, base * scale, scores, iou_threshold=0.5, score_threshold=0.1)
    mixed = base.clone()
    mixed[0, ::3] *= 1e15
    run_both(capi, mixed, scores, iou_threshold=0.4, score_threshold=0.1)
    for thr in (0.0, -0.5, 1e-7, 1e-30, 5.0):
        run_both(capi, base, scores, iou_threshold=thr, score_threshold=0.1)
    odd = base.clone()
    odd[0, 3, 0] = float("nan")
    odd[0, 10, 2] = float("inf")
    odd[0, 17] = torch.tensor([float("-inf"), 0.0, float("inf"), 5.0])
    odd[0, 21, 3] = float("nan")
    run_both(capi, odd, scores, iou_threshold=0.5, score_threshold=0.1)


def test_candidate_counts_around_the_sort_limits(capi):
    """Lists of 511 .. 513 candidates (register sort / shared-memory sort), an odd number of ordered boxes (the mask
    takes rows in pairs), lists cut down before the sort, and all scores tied (the cut then reaches the index bits)."""
    g = torch.Generator().manual_seed(46)
    for N in (127, 128, 129, 511, 512, 513):
        xy = torch.rand(1, N, 2, generator=g) * 200
        wh = torch.rand(1, N, 2, generator=g) * 30 + 1
        boxes = torch.cat([xy, xy + wh], -1)
        scores = torch.rand(1, 2, N, generator=g) * 0.9 + 0.1
        run_both(capi, boxes, scores, iou_threshold=0.5, score_threshold=0.05)
    N = 1000
    xy = torch.rand(1, N, 2, generator=g) * 300
    wh = torch.rand(1, N, 2, generator=g) * 40 + 1
    boxes = torch.cat([xy, xy + wh], -1)
    scores = torch.rand(1, 3, N, generator=g) * 0.9 + 0.1
    for pre in (256, 300, 301, 511, 512):
        run_both(capi, boxes, scores, iou_threshold=0.5, score_threshold=0.05, pre_topk=pre)
    tied = torch.full((1, 2, N), 0.5)
    tied[0, 1, ::2] = 0.75
    for pre in (100, 301):
        run_both(capi, boxes, tied, iou_threshold=0.5, score_threshold=0.05, pre_topk=pre)
    # more candidates than scan slots (1024) and a tie across the cut
    N = 1500
    xy = torch.rand(1, N, 2, generator=g) * 300
    boxes = torch.cat([xy, xy + 20], -1)
    tied = torch.full((1, 1, N), 0.5)
    run_both(capi, boxes, tied, iou_threshold=0.5, score_threshold=0.05, pre_topk=300)


def test_capacity_and_repeat(capi):
    boxes, scores = workloads.yolo_detect(batch=1, classes=4)
    kw = dict(workloads.YOLO_PARAMS)
    rows, count = capi.nms(boxes.cuda(), scores.cuda(), capacity_rows=10, **kw)
    want_rows, total, _ = oracle.nms(boxes.numpy(), scores.numpy(), **kw)
    assert int(count.item()) == total and total > 10
    assert np.array_equal(rows[:10].cpu().numpy(), want_rows[:10])
    # the same workspace serves consecutive calls
    d = capi.NmsDesc(num_batch=1, num_class=4, num_boxes=8400, center_point_box=1, max_output_boxes_per_class=300,
                     pre_topk=300, iou_threshold=0.45, score_threshold=0.25, capacity_rows=1200)
    ws = capi.Workspace(capi.nms_workspace_bytes(d))
    a = capi.nms(boxes.cuda(), scores.cuda(), workspace=ws, **kw)
    b = capi.nms(boxes.cuda(), scores.cuda(), workspace=ws, **kw)
    assert torch.equal(a[0][:total], b[0][:total]) and int(b[1].item()) == total


def test_argument_errors(capi):
    import ctypes as C
    L = capi.lib()
    d = capi.NmsDesc(num_batch=1, num_class=1, num_boxes=10000, center_point_box=0, max_output_boxes_per_class=0,
                     pre_topk=0, iou_threshold=0.5, score_threshold=0.1, capacity_rows=10)
    n = C.c_size_t()
    assert L.vkop_cuda_nms_workspace(C.byref(d), C.byref(n)) == capi.UNSUPPORTED  # too many boxes without pre_topk
    d.num_boxes = -1
    assert L.vkop_cuda_nms_workspace(C.byref(d), C.byref(n)) == capi.INVALID_ARG
    assert L.vkop_cuda_nms(None, None, None, None, None, None, 0, None) == capi.INVALID_ARG


def _head(boxes: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
    """The layout a YOLO-style detection head emits: [B, 4 + C, N], coordinate planes first."""
    return torch.cat([boxes.transpose(1, 2), scores], dim=1).contiguous()


@pytest.mark.parametrize("batch,classes,anchors", [(2, 12, 8400), (3, 5, 1001), (1, 1, 37), (16, 80, 8400)])
def test_nms_on_the_detection_head_in_place(capi, batch, classes, anchors):
    """vkop_cuda_yolo_nms reads boxes and scores where the head holds them; the result must be the rows
    vkop_cuda_nms gives on the separate tensors, which the oracle pins."""
    boxes, scores = workloads.yolo_detect(seed=21, batch=batch, classes=classes, anchors=anchors)
    kw = dict(workloads.YOLO_PARAMS)
    if anchors < 300:
        kw["pre_topk"] = 0
    want_rows, want_total, _ = oracle.nms(boxes.numpy(), scores.numpy(), **kw)
    rows, count = capi.yolo_nms(_head(boxes, scores).cuda(), **kw)
    torch.cuda.synchronize()
    n = int(count.item())
    assert n == want_total
    got = rows[:min(n, rows.shape[0])].cpu().numpy()
    assert np.array_equal(got, want_rows[:got.shape[0]])
    # an odd offset of the head inside its buffer: the score planes no longer start on 16 bytes
    buf = torch.zeros(_head(boxes, scores).numel() + 3)
    buf[1:-2] = _head(boxes, scores).flatten()
    shifted = buf.cuda()[1:-2].view(batch, 4 + classes, anchors)
    rows2, count2 = capi.yolo_nms(shifted, **kw)
    torch.cuda.synchronize()
    assert int(count2.item()) == want_total
    assert np.array_equal(rows2[:got.shape[0]].cpu().numpy(), got)
