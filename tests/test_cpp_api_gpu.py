"""The C++ operator API (host-side mirror of the reference's Operator / Runtime interface) on a GPU."""
from __future__ import annotations

import ctypes
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "op_api_test")
HOST_LIB = os.path.join(ROOT, "vkop_b200", "libvkop_host.so")


def test_host_library_exports():
    """No GPU needed: the host library loads and exports its flat entry points."""
    assert os.path.exists(HOST_LIB), "build it with `python -m vkop_b200.build`"
    lib = ctypes.CDLL(HOST_LIB)
    for name in ("vkop_host_pipeline_create", "vkop_host_pipeline_run", "vkop_host_pipeline_destroy", "vkop_host_last_error",
                 "vkop_host_model_describe", "vkop_host_model_run"):
        assert hasattr(lib, name), name


@pytest.mark.gpu
def test_operator_api_program():
    """tests/cpp/op_api_test.cpp: TopK / Softmax / Nms through create_from_type + onExecute, and the
    RegisterPostProcess pipeline of the reference's benchmark, each compared with the oracle."""
    assert os.path.exists(BIN), "build it with `python -m vkop_b200.build`"
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "all operator API cases passed" in r.stdout


@pytest.mark.gpu
def test_host_pipeline_from_python():
    import numpy as np
    import torch

    import oracle
    from vkop_b200 import workloads

    from vkop_b200 import host_api

    x = workloads.llm_vocab(rows=8)
    xa = x.numpy()
    for fuse in (True, False):
        pipe = host_api.HostPipeline(0, 8, xa.shape[1], 0, 50, 1.0, fuse)
        vals = np.empty((8, 50), np.float32)
        idx = np.empty((8, 50), np.int32)
        assert pipe.run(xa, vals, idx) >= 0.0
        pipe.close()
        wv, wi = oracle.softmax_topk(xa, 50)
        assert np.array_equal(idx, wi)
        assert np.all(np.abs(vals - wv) <= 1e-6 + 1e-5 * np.abs(wv))
