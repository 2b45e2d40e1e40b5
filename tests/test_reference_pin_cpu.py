"""CPU tests that pin the oracle to the REFERENCE'S OWN CPU code for this path.

Two layers: (1) the stored outputs of that code (tests/golden/reference_code_outputs.npz, made by
tests/golden/make_reference_golden.py where the reference checkout is mounted) -- always run; (2) the compiled
functions themselves (oracle/_ref, built by oracle/build_ref.py) on more inputs -- run where they exist."""
from __future__ import annotations

import os

import numpy as np
import pytest

import oracle
from oracle import ref
from vkop_b200 import workloads

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def stored():
    return np.load(os.path.join(GOLDEN, "reference_code_outputs.npz"))


def corners_of(cxcywh: np.ndarray) -> np.ndarray:
    h = np.float32(0.5)
    return np.stack([cxcywh[..., 0] - cxcywh[..., 2] * h, cxcywh[..., 1] - cxcywh[..., 3] * h,
                     cxcywh[..., 0] + cxcywh[..., 2] * h, cxcywh[..., 1] + cxcywh[..., 3] * h], -1).astype(np.float32)


def test_stored_topk_of_the_reference_test_helper(stored):
    """tests/TopkTest.cpp get_top_k_predictions on the seed-56 cases: indices and values bit for bit."""
    g = np.load(os.path.join(GOLDEN, "topk_seed56.npz"))
    for n in range(5):
        v, i = oracle.topk(g[f"case{n}_f32_input"], int(g[f"case{n}_k"]))
        assert np.array_equal(i, stored[f"topk{n}_indices"]) and np.array_equal(v, stored[f"topk{n}_values"])


def test_stored_softmax_of_the_reference_test_helper(stored):
    """tests/SoftmaxTest.cpp softmax_nd on the seed-42 cases, every axis: bit for bit with the sequential fp32 sum."""
    g = np.load(os.path.join(GOLDEN, "softmax_seed42.npz"))
    for n in range(6):
        y = oracle.softmax(g[f"case{n}_f32_input"], int(g[f"case{n}_axis"]), sum_mode=oracle.SUM_F32_SEQUENTIAL)
        assert np.array_equal(y, stored[f"softmax{n}_output"])


def test_stored_nms_expectation_of_the_reference_test(stored):
    """tests/NmsTest.cpp compute_expected_nms on the three test cases and on one image of the detect configuration."""
    g = np.load(os.path.join(GOLDEN, "nms_cases.npz"))
    for n in range(3):
        _, iou, sc = g[f"case{n}_params"]
        rows, total, _ = oracle.nms(g[f"case{n}_boxes"], g[f"case{n}_scores"], iou_threshold=float(iou), score_threshold=float(sc))
        assert np.array_equal(rows[:total], stored[f"nms{n}_rows"])
    boxes, scores = workloads.yolo_detect(batch=1, classes=4)
    rows, total, _ = oracle.nms(boxes.numpy(), scores.numpy(), center_point_box=1,
                                iou_threshold=workloads.YOLO_PARAMS["iou_threshold"],
                                score_threshold=workloads.YOLO_PARAMS["score_threshold"])
    assert np.array_equal(rows[:total], stored["c4_rows"])


def test_stored_function_get_top_k_predictions(stored):
    """core/function.cpp Function::get_top_k_predictions on the classifier and vocabulary configurations."""
    x = workloads.classifier_head().numpy()
    v, i = oracle.softmax_topk(x, 5, sum_mode=oracle.SUM_F32_SEQUENTIAL)
    assert np.array_equal(i, stored["c1_indices"]) and np.array_equal(v, stored["c1_probs"])
    x = workloads.llm_vocab(rows=stored["c3_indices"].shape[0]).numpy()
    v, i = oracle.softmax_topk(x, workloads.LLM_K, workloads.LLM_INV_TEMPERATURE, sum_mode=oracle.SUM_F32_SEQUENTIAL)
    assert np.array_equal(i, stored["c3_indices"]) and np.array_equal(v, stored["c3_probs"])
    # Rows with ties: the probabilities agree bit for bit; std::sort leaves the order of equal probabilities
    # unspecified, so indices are compared where the k + 1 best probabilities of the row are distinct.
    x = workloads.batched_classifier().numpy()
    v, i = oracle.softmax_topk(x, 5, sum_mode=oracle.SUM_F32_SEQUENTIAL)
    assert np.array_equal(v, stored["c2_probs"])
    v6, _ = oracle.softmax_topk(x, 6, sum_mode=oracle.SUM_F32_SEQUENTIAL)
    distinct = (np.diff(v6, axis=1) != 0).all(axis=1)
    assert distinct.sum() >= 200
    assert np.array_equal(i[distinct], stored["c2_indices"][distinct])


needs_ref = pytest.mark.skipif(not ref.available(), reason="oracle/_ref is not built and no reference checkout is mounted")


@needs_ref
def test_compiled_reference_code_on_more_inputs():
    """The compiled reference functions against the oracle on fresh seeded inputs (any axis, any shape)."""
    rng = np.random.default_rng(81)
    for shape, axis in [((3, 5, 7, 2), 0), ((2, 9, 4, 4), 1), ((1, 3, 17, 5), 2), ((4, 2, 3, 33), 3), ((6, 777), 1), ((6, 777), 0)]:
        x = rng.standard_normal(shape).astype(np.float32) * 4
        assert np.array_equal(ref.softmax_nd(x, axis), oracle.softmax(x, axis, sum_mode=oracle.SUM_F32_SEQUENTIAL))
    for rows, cols, k in [(5, 1000, 10), (2, 70001, 50), (16, 4096, 1), (3, 300, 255)]:
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        i, v = ref.topk_rows(x, k)
        ov, oi = oracle.topk(x, k)
        assert np.array_equal(i, oi) and np.array_equal(v, ov)
        for inv_t in (1.0, 1.25):
            i, p = ref.function_top_k_predictions(x, k, inv_t)
            ov, oi = oracle.softmax_topk(x, k, inv_t, sum_mode=oracle.SUM_F32_SEQUENTIAL)
            # selection on rounded probabilities (the reference) and on the logits (the oracle) agree wherever the
            # best k + 1 probabilities are distinct
            if k < cols:
                v1, _ = oracle.softmax_topk(x, k + 1, inv_t, sum_mode=oracle.SUM_F32_SEQUENTIAL)
                distinct = (np.diff(v1, axis=1) != 0).all(axis=1)
            else:
                distinct = np.ones(rows, bool)
            assert np.array_equal(p, ov)
            assert np.array_equal(i[distinct], oi[distinct])


@pytest.mark.skipif(not ref.available(nms=True), reason="oracle/_ref (NMS part) is not built and no reference checkout is mounted")
def test_compiled_reference_nms_on_more_inputs():
    rng = np.random.default_rng(82)
    for B, Cn, N, iou, sc in [(2, 3, 120, 0.5, 0.3), (1, 1, 400, 0.3, 0.1), (3, 2, 64, 0.7, 0.6)]:
        scores = rng.random((B, Cn, N), dtype=np.float32)
        c = rng.random((B, N, 2), dtype=np.float32)
        s = rng.random((B, N, 2), dtype=np.float32) * np.float32(0.6)
        boxes = np.concatenate([c - s / 2, c + s / 2], -1).astype(np.float32)
        want = ref.nms_expected(boxes, scores, iou, sc)
        rows, total, _ = oracle.nms(boxes, scores, iou_threshold=iou, score_threshold=sc)
        assert np.array_equal(rows[:total], want)
