"""Generates ``reference_code_outputs.npz``: outputs of the REFERENCE'S OWN CPU code for this path.

``oracle/build_ref.py`` compiles four functions out of the reference checkout (core/function.cpp
Function::get_top_k_predictions, tests/SoftmaxTest.cpp softmax_nd, tests/TopkTest.cpp get_top_k_predictions,
tests/NmsTest.cpp NmsTest::compute_expected_nms); this script runs them on the inputs of the other fixtures of
this directory and on the benchmark configurations' synthetic inputs, and stores what they return.  The stored
vectors travel to machines that hold no reference checkout; ``tests/test_reference_pin_cpu.py`` checks the CPU
oracle against them (and against the compiled functions themselves where those are present).

Run where the reference checkout is mounted:  python tests/golden/make_reference_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import build_ref, ref  # noqa: E402
from vkop_b200 import workloads  # noqa: E402

LLM_ROWS = 8  # rows of the 64 x 128256 configuration that are stored


def main():
    assert build_ref.reference_present(), "the reference checkout is needed to (re)generate this fixture"
    build_ref.build(force=True)
    out = {}
    with open(os.path.join(build_ref.OUT, "EXTRACTED_FROM.txt")) as f:
        out["extracted_from"] = np.array(f.read())
    g = np.load(os.path.join(HERE, "topk_seed56.npz"))
    for n in range(5):
        i, v = ref.topk_rows(g[f"case{n}_f32_input"], int(g[f"case{n}_k"]))
        out[f"topk{n}_indices"], out[f"topk{n}_values"] = i, v
    g = np.load(os.path.join(HERE, "softmax_seed42.npz"))
    for n in range(6):
        out[f"softmax{n}_output"] = ref.softmax_nd(g[f"case{n}_f32_input"], int(g[f"case{n}_axis"]))
    g = np.load(os.path.join(HERE, "nms_cases.npz"))
    for n in range(3):
        _, iou, sc = g[f"case{n}_params"]
        out[f"nms{n}_rows"] = ref.nms_expected(g[f"case{n}_boxes"], g[f"case{n}_scores"], float(iou), float(sc))
    # the benchmark configurations (inputs are regenerated from their seeds by the test)
    i, p = ref.function_top_k_predictions(workloads.classifier_head().numpy(), 5)
    out["c1_indices"], out["c1_probs"] = i, p
    i, p = ref.function_top_k_predictions(workloads.batched_classifier().numpy(), 5)
    out["c2_indices"], out["c2_probs"] = i, p
    x = workloads.llm_vocab(rows=LLM_ROWS).numpy()
    i, p = ref.function_top_k_predictions(x, workloads.LLM_K, workloads.LLM_INV_TEMPERATURE)
    out["c3_indices"], out["c3_probs"] = i, p
    boxes, scores = workloads.yolo_detect(batch=1, classes=4)
    cxcywh = boxes.numpy()
    corners = np.stack([cxcywh[..., 0] - cxcywh[..., 2] * np.float32(0.5), cxcywh[..., 1] - cxcywh[..., 3] * np.float32(0.5),
                        cxcywh[..., 0] + cxcywh[..., 2] * np.float32(0.5), cxcywh[..., 1] + cxcywh[..., 3] * np.float32(0.5)],
                       -1).astype(np.float32)
    out["c4_rows"] = ref.nms_expected(corners, scores.numpy(), workloads.YOLO_PARAMS["iou_threshold"],
                                      workloads.YOLO_PARAMS["score_threshold"])
    path = os.path.join(HERE, "reference_code_outputs.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
