"""Seeded synthetic inputs with the shapes and value distributions of the
post-processing workloads (classifier heads, an LLM vocabulary head, a YOLO
detect head).  Generated with torch's CPU generator so that the same tensors
can be rebuilt wherever torch is installed; they stand in for the model
outputs the reference's benchmark and examples would produce.
"""
from __future__ import annotations

import torch


def classifier_head(seed: int = 0) -> torch.Tensor:
    """fp32 logits [1, 1000] ~ N(0, 3^2)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, 1000, generator=g) * 3


def batched_classifier(seed: int = 1, rows: int = 256, cols: int = 1000) -> torch.Tensor:
    """fp32 logits [256, 1000] ~ N(0, 3^2); every 8th row quantised to multiples of 1/64 (forces ties)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * 3
    x[::8] = torch.round(x[::8] * 64) / 64
    return x


def spiked_normal(rows: int, cols: int, spikes: int, spike_mean: float, std: float, seed: int,
                  dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """N(0, std^2) logits with `spikes` entries per row overwritten by N(spike_mean, 1)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    if std != 1.0:
        x *= std
    idx = torch.randint(0, cols, (rows, spikes), generator=g)
    s = torch.randn(rows, spikes, generator=g) + spike_mean
    x.scatter_(1, idx, s)
    return x.to(dtype)


def llm_vocab(seed: int = 2, rows: int = 64, cols: int = 128256, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """logits [64, 128256] ~ N(0,1) + 20 spikes/row ~ N(8,1); used with temperature 0.8 and k = 50."""
    return spiked_normal(rows, cols, 20, 8.0, 1.0, seed, dtype)


LLM_INV_TEMPERATURE = 1.25  # 1 / 0.8 evaluated in fp32
LLM_K = 50


def sharded_vocab(seed: int = 4, rows: int = 512, cols: int = 256000) -> torch.Tensor:
    """bf16 logits [512, 256000] ~ N(0, 1.5^2) + 32 spikes/row ~ N(9,1); k = 64."""
    return spiked_normal(rows, cols, 32, 9.0, 1.5, seed, torch.bfloat16)


def long_row(seed: int = 5, cols: int = 16777216) -> torch.Tensor:
    """one fp32 row of 16,777,216 elements ~ N(0,1); k = 1024."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, cols, generator=g)


def yolo_detect(seed: int = 3, batch: int = 16, classes: int = 80, anchors: int = 8400):
    """scores [B, C, N] = sigmoid(N(-4, 2^2)); boxes [B, N, 4] = (cx, cy, w, h) with cx,cy ~ U(0,640),
    w,h ~ U(4,320).  Used with center_point_box = 1, score threshold 0.25, per-class top-300 preselect,
    IoU 0.45, at most 300 kept per class."""
    g = torch.Generator().manual_seed(seed)
    scores = torch.sigmoid(torch.randn(batch, classes, anchors, generator=g) * 2 - 4)
    cxcy = torch.rand(batch, anchors, 2, generator=g) * 640
    wh = torch.rand(batch, anchors, 2, generator=g) * 316 + 4
    boxes = torch.cat([cxcy, wh], -1).contiguous()
    return boxes, scores


YOLO_PARAMS = dict(center_point_box=1, score_threshold=0.25, pre_topk=300, iou_threshold=0.45,
                   max_output_boxes_per_class=300)
