"""ctypes binding of the C ABI declared in ``include/vkop_cuda.h``.

The wrappers take torch CUDA tensors (device memory only; nothing is computed
by torch) and enqueue on torch's current stream.  A missing or unloadable
``libvkop_cuda.so`` raises; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvkop_cuda.so")

F32, F16, BF16 = 0, 1, 2
I32, I64 = 0, 1
VALUE_PROBABILITY, VALUE_RAW = 0, 1
PATH_AUTO, PATH_CHUNK, PATH_RADIX, PATH_STREAM, PATH_BULK = 0, 1, 2, 3, 4
FLAG_INPUT_READY = 1
OK, INVALID_ARG, UNSUPPORTED, WORKSPACE_TOO_SMALL, CUDA_ERROR, TIMEOUT = 0, -1, -2, -3, -4, -5

EXPORTS = [
    "vkop_cuda_version", "vkop_cuda_status_string", "vkop_cuda_launch_count", "vkop_cuda_workspace_init",
    "vkop_cuda_softmax_topk_workspace", "vkop_cuda_softmax_topk", "vkop_cuda_topk", "vkop_cuda_softmax",
    "vkop_cuda_packet_bytes", "vkop_cuda_softmax_topk_partial", "vkop_cuda_softmax_topk_merge",
    "vkop_cuda_nms_workspace", "vkop_cuda_nms",
    "vkop_cuda_static_scratch_bytes", "vkop_cuda_softmax_topk_static",
    "vkop_cuda_packets_push", "vkop_cuda_packets_wait", "vkop_cuda_packets_exchange_all_ranks", "vkop_cuda_yolo_nms",
    "vkop_cuda_sample_topk", "vkop_cuda_topk_axis_workspace", "vkop_cuda_topk_axis",
]


class SoftmaxTopkDesc(C.Structure):
    _fields_ = [("rows", C.c_int64), ("cols", C.c_int64), ("row_stride", C.c_int64), ("dtype", C.c_int32),
                ("k", C.c_int32), ("index_dtype", C.c_int32), ("value_kind", C.c_int32),
                ("inv_temperature", C.c_float), ("largest", C.c_int32), ("path", C.c_int32), ("splits", C.c_int32),
                ("index_offset", C.c_int64), ("flags", C.c_int32), ("reserved", C.c_int32)]


class SoftmaxDesc(C.Structure):
    _fields_ = [("outer", C.c_int64), ("axis_len", C.c_int64), ("inner", C.c_int64), ("dtype", C.c_int32),
                ("inv_temperature", C.c_float)]


class TopkAxisDesc(C.Structure):
    _fields_ = [("outer", C.c_int64), ("axis_len", C.c_int64), ("inner", C.c_int64), ("dtype", C.c_int32),
                ("k", C.c_int32), ("index_dtype", C.c_int32), ("largest", C.c_int32), ("sorted", C.c_int32),
                ("path", C.c_int32)]


class NmsDesc(C.Structure):
    _fields_ = [("num_batch", C.c_int32), ("num_class", C.c_int32), ("num_boxes", C.c_int32),
                ("center_point_box", C.c_int32), ("max_output_boxes_per_class", C.c_int32), ("pre_topk", C.c_int32),
                ("iou_threshold", C.c_float), ("score_threshold", C.c_float), ("capacity_rows", C.c_int64)]


class VkopError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} ({status})")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m vkop_b200.build` "
                               "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        L.vkop_cuda_status_string.restype = C.c_char_p
        L.vkop_cuda_launch_count.restype = C.c_uint64
        L.vkop_cuda_packet_bytes.restype = C.c_size_t
        L.vkop_cuda_packet_bytes.argtypes = [C.c_int32]
        vp, sz = C.c_void_p, C.c_size_t
        L.vkop_cuda_workspace_init.argtypes = [vp, sz, vp]
        L.vkop_cuda_softmax_topk_workspace.argtypes = [C.POINTER(SoftmaxTopkDesc), C.POINTER(sz)]
        L.vkop_cuda_softmax_topk.argtypes = [C.POINTER(SoftmaxTopkDesc), vp, vp, vp, vp, sz, vp]
        L.vkop_cuda_topk.argtypes = [C.POINTER(SoftmaxTopkDesc), vp, vp, vp, vp, sz, vp]
        L.vkop_cuda_softmax.argtypes = [C.POINTER(SoftmaxDesc), vp, vp, vp]
        L.vkop_cuda_topk_axis_workspace.argtypes = [C.POINTER(TopkAxisDesc), C.POINTER(sz)]
        L.vkop_cuda_topk_axis.argtypes = [C.POINTER(TopkAxisDesc), vp, vp, vp, vp, sz, vp]
        L.vkop_cuda_softmax_topk_partial.argtypes = [C.POINTER(SoftmaxTopkDesc), vp, vp, vp, sz, vp]
        L.vkop_cuda_softmax_topk_merge.argtypes = [C.POINTER(SoftmaxTopkDesc), vp, C.c_int32, vp, vp, vp]
        L.vkop_cuda_nms_workspace.argtypes = [C.POINTER(NmsDesc), C.POINTER(sz)]
        L.vkop_cuda_nms.argtypes = [C.POINTER(NmsDesc), vp, vp, vp, vp, vp, sz, vp]
        L.vkop_cuda_packets_push.argtypes = [vp, sz, vp, vp, C.c_int32, C.c_int32, C.c_uint32, vp, vp]
        L.vkop_cuda_packets_wait.argtypes = [vp, C.c_int32, C.c_uint32, C.c_uint32, vp, vp]
        L.vkop_cuda_packets_exchange_all_ranks.argtypes = [vp, sz, vp, vp, C.c_int32, C.c_uint32, vp, C.c_uint32, vp, vp]
        L.vkop_cuda_yolo_nms.argtypes = [C.POINTER(NmsDesc), vp, vp, vp, vp, sz, vp]
        L.vkop_cuda_sample_topk.argtypes = [vp, C.c_int32, vp, C.c_int32, C.c_int64, C.c_int32, C.c_float, vp, vp, vp, vp]
        L.vkop_cuda_static_scratch_bytes.restype = sz
        L.vkop_cuda_softmax_topk_static.argtypes = [C.POINTER(SoftmaxTopkDesc), vp, vp, vp, vp]
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().vkop_cuda_status_string(C.c_int(status)).decode()


def launch_count() -> int:
    return int(lib().vkop_cuda_launch_count())


def check(status: int, where: str) -> None:
    if status != OK:
        raise VkopError(status, where)


_TORCH_DTYPE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def dtype_tag(t: torch.Tensor) -> int:
    return _TORCH_DTYPE[t.dtype]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


class Workspace:
    """Caller-owned scratch memory (a torch byte tensor), cleared once on creation."""

    def __init__(self, nbytes: int, device="cuda"):
        self.nbytes = int(nbytes)
        self.buf = torch.empty(max(self.nbytes, 16), dtype=torch.uint8, device=device)
        check(lib().vkop_cuda_workspace_init(self.buf.data_ptr(), self.buf.numel(), _stream()), "workspace_init")

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()


def make_desc(logits: torch.Tensor, k: int, inv_temperature: float = 1.0, index_dtype: int = I32,
              value_kind: int = VALUE_PROBABILITY, largest: bool = True, path: int = PATH_AUTO, splits: int = 0,
              index_offset: int = 0, flags: int = 0) -> SoftmaxTopkDesc:
    assert logits.dim() == 2 and logits.stride(1) == 1
    return SoftmaxTopkDesc(rows=logits.shape[0], cols=logits.shape[1], row_stride=logits.stride(0),
                           dtype=dtype_tag(logits), k=k, index_dtype=index_dtype, value_kind=value_kind,
                           inv_temperature=inv_temperature, largest=int(largest), path=path, splits=splits,
                           index_offset=index_offset, flags=flags, reserved=0)


def softmax_topk_workspace_bytes(desc: SoftmaxTopkDesc) -> int:
    n = C.c_size_t(0)
    check(lib().vkop_cuda_softmax_topk_workspace(C.byref(desc), C.byref(n)), "softmax_topk_workspace")
    return int(n.value)


def softmax_topk(logits: torch.Tensor, k: int, inv_temperature: float = 1.0, index_dtype: int = I32,
                 value_kind: int = VALUE_PROBABILITY, path: int = PATH_AUTO, splits: int = 0, index_offset: int = 0,
                 workspace: Workspace | None = None, out=None, standalone_topk: bool = False, largest: bool = True,
                 flags: int = 0):
    """Fused softmax + top-k of a 2-D CUDA tensor.  Returns (values [rows,k] in the logits dtype, indices)."""
    if not logits.is_cuda:
        raise RuntimeError("vkop_b200 runs on CUDA device memory only")
    desc = make_desc(logits, k, inv_temperature, index_dtype, value_kind, largest, path, splits, index_offset, flags)
    need = softmax_topk_workspace_bytes(desc)
    if workspace is None or workspace.nbytes < need:
        workspace = Workspace(need, logits.device)
    if out is None:
        values = torch.empty((logits.shape[0], k), dtype=logits.dtype, device=logits.device)
        indices = torch.empty((logits.shape[0], k), dtype=torch.int64 if index_dtype == I64 else torch.int32,
                              device=logits.device)
    else:
        values, indices = out
    fn = lib().vkop_cuda_topk if standalone_topk else lib().vkop_cuda_softmax_topk
    check(fn(C.byref(desc), logits.data_ptr(), values.data_ptr(), indices.data_ptr(), workspace.ptr,
             workspace.buf.numel(), _stream()), "topk" if standalone_topk else "softmax_topk")
    return values, indices


def topk_axis(x: torch.Tensor, k: int, axis: int = -1, largest: bool = True, sorted: bool = True, index_dtype: int = I32,
              path: int = PATH_AUTO, workspace: Workspace | None = None):
    """TopK of a contiguous CUDA tensor along any axis.  Returns (values, indices) shaped like x with shape[axis] = k;
    sorted=False gives the k entries in ascending index order."""
    if not x.is_cuda or not x.is_contiguous():
        raise RuntimeError("vkop_b200 runs on contiguous CUDA device memory only")
    axis = axis % x.dim()
    outer = int(torch.Size(x.shape[:axis]).numel())
    inner = int(torch.Size(x.shape[axis + 1:]).numel())
    desc = TopkAxisDesc(outer=outer, axis_len=x.shape[axis], inner=inner, dtype=dtype_tag(x), k=k, index_dtype=index_dtype,
                        largest=int(largest), sorted=int(sorted), path=path)
    n = C.c_size_t(0)
    check(lib().vkop_cuda_topk_axis_workspace(C.byref(desc), C.byref(n)), "topk_axis_workspace")
    if workspace is None or workspace.nbytes < n.value:
        workspace = Workspace(int(n.value), x.device)
    shape = list(x.shape)
    shape[axis] = k
    values = torch.empty(shape, dtype=x.dtype, device=x.device)
    indices = torch.empty(shape, dtype=torch.int64 if index_dtype == I64 else torch.int32, device=x.device)
    check(lib().vkop_cuda_topk_axis(C.byref(desc), x.data_ptr(), values.data_ptr(), indices.data_ptr(), workspace.ptr,
                                    workspace.buf.numel(), _stream()), "topk_axis")
    return values, indices


def yolo_nms(head: torch.Tensor, center_point_box: int = 1, max_output_boxes_per_class: int = 0,
             iou_threshold: float = 0.0, score_threshold: float = 0.0, pre_topk: int = 0, capacity_rows: int | None = None,
             workspace: Workspace | None = None, out=None):
    """NMS on a detection head [B, 4 + C, N] (coordinate planes, then score planes), read in place.
    Returns (rows int32 [capacity, 3], count int32 [1]) like nms()."""
    if not head.is_cuda:
        raise RuntimeError("vkop_b200 runs on CUDA device memory only")
    assert head.dtype == torch.float32 and head.dim() == 3 and head.shape[1] > 4 and head.is_contiguous()
    B, planes, N = head.shape
    Cn = planes - 4
    if capacity_rows is None:
        per = max_output_boxes_per_class if max_output_boxes_per_class > 0 else (pre_topk if pre_topk > 0 else N)
        capacity_rows = B * Cn * min(per, N)
    desc = NmsDesc(num_batch=B, num_class=Cn, num_boxes=N, center_point_box=center_point_box,
                   max_output_boxes_per_class=max_output_boxes_per_class, pre_topk=pre_topk,
                   iou_threshold=iou_threshold, score_threshold=score_threshold, capacity_rows=capacity_rows)
    need = nms_workspace_bytes(desc)
    if workspace is None or workspace.nbytes < need:
        workspace = Workspace(need, head.device)
    if out is None:
        rows = torch.empty((max(capacity_rows, 1), 3), dtype=torch.int32, device=head.device)
        count = torch.empty(1, dtype=torch.int32, device=head.device)
    else:
        rows, count = out
    check(lib().vkop_cuda_yolo_nms(C.byref(desc), head.data_ptr(), rows.data_ptr(), count.data_ptr(), workspace.ptr,
                                   workspace.buf.numel(), _stream()), "yolo_nms")
    return rows, count


def sample_topk(values: torch.Tensor, indices: torch.Tensor, top_p: float, u: torch.Tensor):
    """Sampling tail over the survivors of softmax_topk.  Returns (choice int32 [rows], token [rows])."""
    if not (values.is_cuda and indices.is_cuda and u.is_cuda):
        raise RuntimeError("vkop_b200 runs on CUDA device memory only")
    rows, k = values.shape
    assert indices.shape == values.shape and u.shape == (rows,) and u.dtype == torch.float32
    values, indices, u = values.contiguous(), indices.contiguous(), u.contiguous()
    choice = torch.empty(rows, dtype=torch.int32, device=values.device)
    token = torch.empty(rows, dtype=indices.dtype, device=values.device)
    check(lib().vkop_cuda_sample_topk(values.data_ptr(), dtype_tag(values), indices.data_ptr(),
                                      I64 if indices.dtype == torch.int64 else I32, rows, k, float(top_p), u.data_ptr(),
                                      choice.data_ptr(), token.data_ptr(), _stream()), "sample_topk")
    return choice, token


def packets_push(packets: torch.Tensor, peer_slots: torch.Tensor, peer_flags: torch.Tensor, rank: int, world: int,
                 seq: int, tickets: torch.Tensor) -> None:
    """peer_slots / peer_flags: int64 CUDA tensors holding one device pointer per rank."""
    check(lib().vkop_cuda_packets_push(packets.data_ptr(), packets.numel() * packets.element_size(), peer_slots.data_ptr(),
                                       peer_flags.data_ptr(), rank, world, seq, tickets.data_ptr(), _stream()), "packets_push")


def packets_wait(flags: torch.Tensor, world: int, seq: int, status: torch.Tensor, max_polls: int = 1 << 20) -> None:
    check(lib().vkop_cuda_packets_wait(flags.data_ptr(), world, seq, max_polls, status.data_ptr(), _stream()), "packets_wait")


def packets_exchange_all_ranks(packet_ptrs: torch.Tensor, packets_bytes: int, peer_slots: torch.Tensor, peer_flags: torch.Tensor,
                               world: int, seq: int, ticket_ptrs: torch.Tensor, status: torch.Tensor, max_polls: int = 1 << 20) -> None:
    """Every rank's push and bounded wait of one step in one cooperative launch (ranks emulated on one GPU).
    packet_ptrs / ticket_ptrs / peer_slots / peer_flags: int64 CUDA tensors of one device pointer per rank."""
    check(lib().vkop_cuda_packets_exchange_all_ranks(packet_ptrs.data_ptr(), packets_bytes, peer_slots.data_ptr(), peer_flags.data_ptr(),
                                                     world, seq, ticket_ptrs.data_ptr(), max_polls, status.data_ptr(), _stream()),
          "packets_exchange_all_ranks")


def static_scratch_bytes() -> int:
    return int(lib().vkop_cuda_static_scratch_bytes())


def softmax_topk_static(logits: torch.Tensor, k: int, inv_temperature: float = 1.0, index_dtype: int = I32,
                        value_kind: int = VALUE_PROBABILITY, out=None):
    """Fused softmax + top-k through the entry point that takes no workspace and allocates nothing
    (the outputs are still the caller's: pass `out`, or they are created here with torch)."""
    if not logits.is_cuda:
        raise RuntimeError("vkop_b200 runs on CUDA device memory only")
    desc = make_desc(logits, k, inv_temperature, index_dtype, value_kind, True, PATH_AUTO, 0, 0, 0)
    if out is None:
        values = torch.empty((logits.shape[0], k), dtype=logits.dtype, device=logits.device)
        indices = torch.empty((logits.shape[0], k), dtype=torch.int64 if index_dtype == I64 else torch.int32,
                              device=logits.device)
    else:
        values, indices = out
    check(lib().vkop_cuda_softmax_topk_static(C.byref(desc), logits.data_ptr(), values.data_ptr(), indices.data_ptr(),
                                              _stream()), "softmax_topk_static")
    return values, indices


def softmax(x: torch.Tensor, axis: int = -1, inv_temperature: float = 1.0) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("vkop_b200 runs on CUDA device memory only")
    x = x.contiguous()
    axis = axis % x.dim()
    outer = 1
    for s in x.shape[:axis]:
        outer *= s
    inner = 1
    for s in x.shape[axis + 1:]:
        inner *= s
    desc = SoftmaxDesc(outer=outer, axis_len=x.shape[axis], inner=inner, dtype=dtype_tag(x),
                       inv_temperature=inv_temperature)
    out = torch.empty_like(x)
    check(lib().vkop_cuda_softmax(C.byref(desc), x.data_ptr(), out.data_ptr(), _stream()), "softmax")
    return out


def packet_bytes(k: int) -> int:
    return int(lib().vkop_cuda_packet_bytes(k))


def softmax_topk_partial(shard: torch.Tensor, k: int, index_offset: int, inv_temperature: float = 1.0,
                         workspace: Workspace | None = None, packets: torch.Tensor | None = None,
                         path: int = PATH_AUTO, splits: int = 0):
    """Per-shard packets [rows, packet_bytes/4] (uint32 words held in an int32 tensor)."""
    desc = make_desc(shard, k, inv_temperature, index_offset=index_offset, path=path, splits=splits)
    need = softmax_topk_workspace_bytes(desc)
    if workspace is None or workspace.nbytes < need:
        workspace = Workspace(need, shard.device)
    if packets is None:
        packets = torch.empty((shard.shape[0], packet_bytes(k) // 4), dtype=torch.int32, device=shard.device)
    check(lib().vkop_cuda_softmax_topk_partial(C.byref(desc), shard.data_ptr(), packets.data_ptr(), workspace.ptr,
                                               workspace.buf.numel(), _stream()), "softmax_topk_partial")
    return packets


def softmax_topk_merge(packets: torch.Tensor, rows: int, k: int, dtype: torch.dtype, inv_temperature: float = 1.0,
                       index_dtype: int = I32, out=None):
    """packets: [shards, rows, words] as gathered.  Returns (values, indices)."""
    shards = packets.shape[0]
    desc = SoftmaxTopkDesc(rows=rows, cols=1, row_stride=0, dtype=_TORCH_DTYPE[dtype], k=k, index_dtype=index_dtype,
                           value_kind=VALUE_PROBABILITY, inv_temperature=inv_temperature, largest=1, path=0, splits=0,
                           index_offset=0)
    if out is None:
        values = torch.empty((rows, k), dtype=dtype, device=packets.device)
        indices = torch.empty((rows, k), dtype=torch.int64 if index_dtype == I64 else torch.int32,
                              device=packets.device)
    else:
        values, indices = out
    check(lib().vkop_cuda_softmax_topk_merge(C.byref(desc), packets.data_ptr(), shards, values.data_ptr(),
                                             indices.data_ptr(), _stream()), "softmax_topk_merge")
    return values, indices


def nms_workspace_bytes(desc: NmsDesc) -> int:
    n = C.c_size_t(0)
    check(lib().vkop_cuda_nms_workspace(C.byref(desc), C.byref(n)), "nms_workspace")
    return int(n.value)


def nms(boxes: torch.Tensor, scores: torch.Tensor, center_point_box: int = 0, max_output_boxes_per_class: int = 0,
        iou_threshold: float = 0.0, score_threshold: float = 0.0, pre_topk: int = 0, capacity_rows: int | None = None,
        workspace: Workspace | None = None, out=None):
    """Returns (rows int32 [capacity,3] device tensor, count int32 [1] device tensor)."""
    if not (boxes.is_cuda and scores.is_cuda):
        raise RuntimeError("vkop_b200 runs on CUDA device memory only")
    B, N, four = boxes.shape
    assert four == 4 and boxes.dtype == torch.float32 and scores.dtype == torch.float32
    Cn = scores.shape[1]
    assert scores.shape[0] == B and scores.shape[2] == N
    boxes, scores = boxes.contiguous(), scores.contiguous()
    if capacity_rows is None:
        per = max_output_boxes_per_class if max_output_boxes_per_class > 0 else (pre_topk if pre_topk > 0 else N)
        capacity_rows = B * Cn * min(per, N)
    desc = NmsDesc(num_batch=B, num_class=Cn, num_boxes=N, center_point_box=center_point_box,
                   max_output_boxes_per_class=max_output_boxes_per_class, pre_topk=pre_topk,
                   iou_threshold=iou_threshold, score_threshold=score_threshold, capacity_rows=capacity_rows)
    need = nms_workspace_bytes(desc)
    if workspace is None or workspace.nbytes < need:
        workspace = Workspace(need, boxes.device)
    if out is None:
        rows = torch.empty((max(capacity_rows, 1), 3), dtype=torch.int32, device=boxes.device)
        count = torch.empty(1, dtype=torch.int32, device=boxes.device)
    else:
        rows, count = out
    check(lib().vkop_cuda_nms(C.byref(desc), boxes.data_ptr(), scores.data_ptr(), rows.data_ptr(), count.data_ptr(),
                              workspace.ptr, workspace.buf.numel(), _stream()), "nms")
    return rows, count
