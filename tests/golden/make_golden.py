"""Generates the golden fixtures in this directory with torch-CPU.

The reference's tests hold no stored vectors: they compute expectations with
libtorch at run time.  This script replays those computations with the
reference's own seeds and shapes and stores inputs and expected outputs, so
that the CPU oracle can be pinned without torch's random stream having to match
across versions.

  topk_seed56.npz     tests/TopkTest.cpp:71-75,93-99   torch.manual_seed(56); randn; torch.topk(largest, sorted)
  softmax_seed42.npz  tests/SoftmaxTest.cpp:118-138,195-202  torch.manual_seed(42); randn; torch.softmax
  nms_cases.npz       tests/NmsTest.cpp:40-56 (box construction), :66-176 (in-test greedy NMS), :181-185 (cases);
                      the reference draws these unseeded, a fixed seed is used here

Run:  python tests/golden/make_golden.py   (torch version is recorded in each file)
"""
from __future__ import annotations

import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

TOPK_CASES = [((1, 200), 7), ((1, 400), 8), ((1, 600), 7), ((3, 2000), 7), ((1, 2000), 6)]
SOFTMAX_CASES = [((1, 10, 7, 7), 1), ((1, 6, 8, 8), 3), ((2, 4, 10, 10), 2), ((1, 8, 6, 6), 2), ((1, 16, 5, 5), 1),
                 ((4, 1000), 1)]
NMS_CASES = [((1, 10, 4), (1, 2, 10), 0, 0.5, 0.5), ((1, 200, 4), (1, 1, 200), 50, 0.7, 0.4),
             ((1, 50, 4), (1, 7, 50), 0, 0.3, 0.2)]


def make_topk():
    out = {"torch_version": np.array(torch.__version__)}
    for n, (shape, k) in enumerate(TOPK_CASES):
        for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
            torch.manual_seed(56)
            x = torch.randn(shape, dtype=dt)
            v, i = torch.topk(x, k, -1, True, True)
            xs = x.numpy()
            vs = v.numpy()
            if dt == torch.float16:
                xs, vs = xs.view(np.uint16), vs.view(np.uint16)
            out[f"case{n}_{tag}_input"] = xs
            out[f"case{n}_{tag}_values"] = vs
            out[f"case{n}_{tag}_indices"] = i.to(torch.int32).numpy()
        out[f"case{n}_k"] = np.array(k)
    np.savez_compressed(os.path.join(HERE, "topk_seed56.npz"), **out)


def make_softmax():
    out = {"torch_version": np.array(torch.__version__)}
    for n, (shape, axis) in enumerate(SOFTMAX_CASES):
        for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
            torch.manual_seed(42)
            x = torch.randn(shape, dtype=dt)
            y = torch.softmax(x, axis)
            xs, ys = x.numpy(), y.numpy()
            if dt == torch.float16:
                xs, ys = xs.view(np.uint16), ys.view(np.uint16)
            out[f"case{n}_{tag}_input"] = xs
            out[f"case{n}_{tag}_output"] = ys
        out[f"case{n}_axis"] = np.array(axis)
    np.savez_compressed(os.path.join(HERE, "softmax_seed42.npz"), **out)


def nms_test_expected(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float, score_threshold: float):
    """The expectation tests/NmsTest.cpp:66-176 computes: per (batch, class) torch.sort descending, keep
    score >= threshold, greedy suppression with clamped intersection sides and union > 1e-8."""
    keep = []
    B, Cn, _ = scores.shape
    for b in range(B):
        for c in range(Cn):
            s, order = torch.sort(scores[b, c], dim=0, descending=True)
            valid = s >= score_threshold
            idx = order[valid]
            if idx.numel() == 0:
                continue
            sel = boxes[b][idx].numpy()
            n = idx.numel()
            dead = [False] * n
            for i in range(n):
                if dead[i]:
                    continue
                keep.append((b, c, int(idx[i])))
                x1i, y1i, x2i, y2i = (np.float32(t) for t in sel[i])
                area_i = np.float32((x2i - x1i) * (y2i - y1i))
                for j in range(i + 1, n):
                    if dead[j]:
                        continue
                    x1j, y1j, x2j, y2j = (np.float32(t) for t in sel[j])
                    w = max(np.float32(0), np.float32(min(x2i, x2j) - max(x1i, x1j)))
                    h = max(np.float32(0), np.float32(min(y2i, y2j) - max(y1i, y1j)))
                    inter = np.float32(w * h)
                    area_j = np.float32((x2j - x1j) * (y2j - y1j))
                    union = np.float32(np.float32(area_i + area_j) - inter)
                    iou = np.float32(inter / union) if union > np.float32(1e-8) else np.float32(0)
                    if iou > np.float32(iou_threshold):
                        dead[j] = True
    return np.array(keep, np.int32).reshape(-1, 3)


def make_nms():
    out = {"torch_version": np.array(torch.__version__)}
    torch.manual_seed(7)
    for n, (bshape, sshape, max_per_class, iou_thr, score_thr) in enumerate(NMS_CASES):
        scores = torch.rand(sshape)
        centre = torch.rand(bshape[0], bshape[1], 2)
        size = torch.rand(bshape[0], bshape[1], 2) * 1.3
        x1 = torch.clamp(centre[..., 0] - size[..., 0] / 2, 0.0, 1.0)
        y1 = torch.clamp(centre[..., 1] - size[..., 1] / 2, 0.0, 1.0)
        x2 = torch.clamp(centre[..., 0] + size[..., 0] / 2, 0.0, 1.0)
        y2 = torch.clamp(centre[..., 1] + size[..., 1] / 2, 0.0, 1.0)
        boxes = torch.stack([x1, y1, x2, y2], -1)
        out[f"case{n}_boxes"] = boxes.numpy()
        out[f"case{n}_scores"] = scores.numpy()
        out[f"case{n}_params"] = np.array([max_per_class, iou_thr, score_thr], np.float64)
        out[f"case{n}_expected"] = nms_test_expected(boxes, scores, iou_thr, score_thr)
    np.savez_compressed(os.path.join(HERE, "nms_cases.npz"), **out)


if __name__ == "__main__":
    make_topk()
    make_softmax()
    make_nms()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
