"""Unfused Softmax (the full probability tensor) on the GPU, through the C ABI: the reference's own test
cases (tests/SoftmaxTest.cpp:195-202: rank-4 NCHW tensors along axes 0-3 and a [4, 1000] matrix, seed 42)
against the stored torch-CPU results and against the oracle, then the shapes of the fused path."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import oracle
from tests import util
from vkop_b200 import workloads

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "softmax_seed42.npz")


@pytest.fixture(scope="module")
def capi():
    from vkop_b200 import capi as c
    return c


def _close(got: torch.Tensor, want: np.ndarray, dtype, what):
    util.assert_probs_close(got, want, dtype, what)


def test_reference_softmax_cases(capi):
    z = np.load(GOLDEN)
    n = len([f for f in z.files if f.endswith("_axis")])
    assert n >= 6
    for c in range(n):
        axis = int(z[f"case{c}_axis"])
        x32 = torch.from_numpy(z[f"case{c}_f32_input"])
        got = capi.softmax(x32.cuda(), axis)
        _close(got, z[f"case{c}_f32_output"], torch.float32, f"case {c} f32 vs torch")
        _close(got, oracle.softmax(x32.numpy(), axis), torch.float32, f"case {c} f32 vs oracle")
        bits = z[f"case{c}_f16_input"]  # fp16 tensors are stored as their uint16 bit patterns
        x16 = torch.from_numpy(bits.view(np.float16))
        got16 = capi.softmax(x16.cuda(), axis)
        assert got16.dtype == torch.float16
        _close(got16, oracle.softmax(bits, axis, dtype=oracle.F16), torch.float16, f"case {c} f16 vs oracle")
        # the stored fp16 result is torch's own rounding of its fp32 math: allow one more rounding step
        want16 = z[f"case{c}_f16_output"].view(np.float16).astype(np.float32)
        assert np.allclose(got16.float().cpu().numpy(), want16, rtol=4e-3, atol=1e-6), f"case {c} f16 vs torch"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_rows_of_the_fused_path(capi, dtype):
    for x in (workloads.classifier_head(), workloads.batched_classifier(rows=64),
              workloads.llm_vocab(rows=6).to(dtype).float(), torch.randn(3, 300007, generator=torch.Generator().manual_seed(5))):
        x = x.to(dtype)
        got = capi.softmax(x.cuda(), -1, 1.25)
        want = oracle.softmax(util.to_oracle_array(x), -1, 1.25, dtype=util.ORACLE_DTYPE[dtype])
        _close(got, want, dtype, f"softmax {tuple(x.shape)} {dtype}")
        s = got.float().sum(-1).cpu()
        assert torch.allclose(s, torch.ones_like(s), atol=2e-2 if dtype != torch.float32 else 1e-4)


def test_every_axis_and_edge_values(capi):
    g = torch.Generator().manual_seed(11)
    x = torch.randn(3, 5, 17, 9, generator=g)
    for axis in range(-4, 4):
        _close(capi.softmax(x.cuda(), axis), oracle.softmax(x.numpy(), axis), torch.float32, f"axis {axis}")
    y = torch.zeros(4, 70000)
    y[1, 5] = float("-inf")
    y[2] = -1e30
    y[3, ::2] = 80.0
    _close(capi.softmax(y.cuda()), oracle.softmax(y.numpy()), torch.float32, "edge values")
    one = torch.randn(7, 1)
    assert torch.equal(capi.softmax(one.cuda()).cpu(), torch.ones(7, 1))
