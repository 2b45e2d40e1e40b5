"""The .vkopbin loader (model/load.cpp:98-285) and Runtime::LoadModel (core/runtime.cpp:33-363) for model files made
of this path's operators.  The parser runs without a GPU; running a loaded model needs one."""
from __future__ import annotations

import ctypes as C
import os
import struct

import numpy as np
import pytest

from tests import vkopbin

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_LIB = os.path.join(ROOT, "vkop_b200", "libvkop_host.so")
REFERENCE_FIXTURE = os.path.join(os.environ.get("VKOP_REFERENCE", "/root/reference"), "model", "add_conv_model.vkopbin")


def host():
    lib = C.CDLL(HOST_LIB)
    lib.vkop_host_model_describe.restype = C.c_long
    lib.vkop_host_model_describe.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
    lib.vkop_host_last_error.restype = C.c_char_p
    lib.vkop_host_model_run.argtypes = [C.c_int, C.c_char_p, C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_size_t),
                                        C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_double)]
    return lib


def describe(lib, path):
    buf = C.create_string_buffer(1 << 16)
    n = lib.vkop_host_model_describe(path.encode(), buf, len(buf))
    if n < 0:
        raise RuntimeError(lib.vkop_host_last_error().decode())
    return buf.value.decode()


def softmax_topk_model(rows, cols, k, k_as_input=False):
    nodes = [dict(op_type="Softmax", name="sm", attrs={"axis": -1}, inputs=[("logits", [rows, cols])],
                  outputs=[("probs", [rows, cols])], dependents=["tk"]),
             dict(op_type="TopK", name="tk", attrs={"axis": -1, "largest": 1, "sorted": 1} if k_as_input else
                  {"k": k, "axis": -1, "largest": 1, "sorted": 1},
                  inputs=[("probs", [rows, cols])] + ([("K", [1])] if k_as_input else []),
                  outputs=[("values", [rows, k]), ("indices", [rows, k])], dependencies=["sm"])]
    inits = [("K", "int64", [1], struct.pack("<q", k))] if k_as_input else []
    return dict(inputs=[("logits", [rows, cols])], outputs=[("values", [rows, k]), ("indices", [rows, k])], nodes=nodes,
                initializers=inits)


def test_parser_reads_what_the_writer_wrote(tmp_path):
    lib = host()
    m = softmax_topk_model(8, 4096, 7, k_as_input=True)
    m["nodes"][0]["attrs"].update({"note": "tail", "scale": 0.5, "pads": [1, 2, 3], "w": [0.25, 1.5]})
    p = str(tmp_path / "tail.vkopbin")
    vkopbin.write_model(p, **m)
    text = describe(lib, p)
    assert "input logits [8,4096]" in text and "output indices [8,7]" in text
    assert "node Softmax sm in logits out probs attrs 5" in text
    assert "node TopK tk in probs K out values indices attrs 3" in text
    assert "initializer K int64 [1] 8" in text and "level 0 sm" in text and "level 1 tk" in text


def test_parser_rejects_truncated_and_missing_files(tmp_path):
    lib = host()
    raw = vkopbin.model_bytes(**softmax_topk_model(2, 100, 3))
    for cut in (3, 20, len(raw) // 2, len(raw) - 1):
        p = str(tmp_path / f"cut{cut}.vkopbin")
        with open(p, "wb") as f:
            f.write(raw[:cut])
        with pytest.raises(RuntimeError):
            describe(lib, p)
    with pytest.raises(RuntimeError):
        describe(lib, str(tmp_path / "absent.vkopbin"))
    p = str(tmp_path / "badtag.vkopbin")
    bad = vkopbin._shapes([("x", [1])]) * 2 + vkopbin._u32(1) + vkopbin._str("Softmax") + vkopbin._str("n") + \
        vkopbin._u32(1) + vkopbin._str("a") + b"\x09"
    with open(p, "wb") as f:
        f.write(bad)
    with pytest.raises(RuntimeError, match="tag"):
        describe(lib, p)


@pytest.mark.skipif(not os.path.exists(REFERENCE_FIXTURE), reason="the reference checkout is not here")
def test_parser_reads_the_reference_fixture():
    """model/add_conv_model.vkopbin, the only model file the reference ships: two inputs, an Add and a Conv node."""
    text = describe(host(), REFERENCE_FIXTURE)
    assert "input input_x1 [1,16,8,8]" in text and "input input_x2 [1,16,8,8]" in text
    assert "node Add " in text and "node Conv " in text and "output output " in text


@pytest.mark.gpu
@pytest.mark.parametrize("k_as_input", [False, True])
def test_loaded_softmax_topk_tail_runs_fused(tmp_path, k_as_input):
    import oracle

    lib = host()
    rows, cols, k = 8, 70000, 7
    p = str(tmp_path / "tail.vkopbin")
    vkopbin.write_model(p, **softmax_topk_model(rows, cols, k, k_as_input))
    rng = np.random.default_rng(5)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    vals = np.empty((rows, k), np.float32)
    idx = np.empty((rows, k), np.int32)
    nv, ni, ms = C.c_size_t(vals.nbytes), C.c_size_t(idx.nbytes), C.c_double()
    rc = lib.vkop_host_model_run(0, p.encode(), x.ctypes.data, x.size, vals.ctypes.data, C.byref(nv), idx.ctypes.data,
                                 C.byref(ni), C.byref(ms))
    assert rc == 0, lib.vkop_host_last_error().decode()
    assert nv.value == vals.nbytes and ni.value == idx.nbytes
    wv, wi = oracle.softmax_topk(x, k)
    assert np.array_equal(idx, wi)
    assert np.all(np.abs(vals - wv) <= 1e-6 + 1e-5 * np.abs(wv))


@pytest.mark.gpu
def test_loaded_nms_node_with_onnx_parameter_inputs(tmp_path):
    """A NonMaxSuppression node on a [B, 4 + C, N] detection head; thresholds arrive as initializers, as ONNX passes them."""
    import oracle
    import torch

    from vkop_b200 import workloads

    lib = host()
    boxes, scores = workloads.yolo_detect(seed=9, batch=2, classes=3, anchors=500)
    head = torch.cat([boxes.transpose(1, 2), scores], 1).contiguous().numpy()  # [B, 4 + C, N]
    B, _, N = head.shape
    node = dict(op_type="NonMaxSuppression", name="nms", attrs={"center_point_box": 1},
                inputs=[("head", [B, 7, N]), ("max_out", [1]), ("iou", [1]), ("score", [1])],
                outputs=[("selected", [B * 3 * N, 3])])
    inits = [("max_out", "int64", [1], struct.pack("<q", 50)), ("iou", "float32", [1], struct.pack("<f", 0.45)),
             ("score", "float32", [1], struct.pack("<f", 0.25))]
    p = str(tmp_path / "nms.vkopbin")
    vkopbin.write_model(p, inputs=[("head", [B, 7, N])], outputs=[("selected", [B * 3 * N, 3])], nodes=[node],
                        initializers=inits)
    want_rows, total, _ = oracle.nms(boxes.numpy(), scores.numpy(), center_point_box=1, max_output_boxes_per_class=50,
                                     iou_threshold=0.45, score_threshold=0.25)
    out = np.full((B * 3 * N, 3), -1, np.int32)
    n0, ms = C.c_size_t(out.nbytes), C.c_double()
    rc = lib.vkop_host_model_run(0, p.encode(), head.ctypes.data, head.size, out.ctypes.data, C.byref(n0), None, None,
                                 C.byref(ms))
    assert rc == 0, lib.vkop_host_last_error().decode()
    assert total > 0 and np.array_equal(out[:total], want_rows)


@pytest.mark.gpu
def test_node_outside_the_path_is_named(tmp_path):
    lib = host()
    node = dict(op_type="Conv", name="conv0", inputs=[("x", [1, 3, 8, 8])], outputs=[("y", [1, 4, 8, 8])])
    p = str(tmp_path / "conv.vkopbin")
    vkopbin.write_model(p, inputs=[("x", [1, 3, 8, 8])], outputs=[("y", [1, 4, 8, 8])], nodes=[node])
    x = np.zeros(192, np.float32)
    rc = lib.vkop_host_model_run(0, p.encode(), x.ctypes.data, x.size, None, None, None, None, None)
    assert rc != 0
    msg = lib.vkop_host_last_error().decode()
    assert "conv0" in msg and "Conv" in msg
