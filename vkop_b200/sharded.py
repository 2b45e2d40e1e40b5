"""Multi-GPU execution of the fused Softmax + TopK: one process per GPU, torch.distributed for the plumbing.

Two ways to shard (the reference runs on a single device; both are extensions of its operator):

* rows     independent rows go to different GPUs; no communication on the data path.
* vocab    every GPU holds one contiguous column slice of all rows.  Each GPU reduces its slice to one packet
           per row (softmax maximum, exp-sum, its k best (key, global index) pairs), the packets are all-gathered
           (NCCL over NVLink), and every GPU merges them: M = max m_g, S = sum s_g * exp(m_g - M), k best of the
           G * k candidates by (key descending, index ascending).  Because a slice's indices are offset by its
           first column, the lower-index-first rule holds across slices.
"""
from __future__ import annotations

import ctypes as _ctypes

import torch
import torch.distributed as dist


def split_even(n: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of the rank-th of `world` contiguous, near-equal parts of n items."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def exchange_packets(packets: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather of the per-row packets: [rows, words] on every rank -> [world, rows, words]."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world,) + tuple(packets.shape), dtype=packets.dtype, device=packets.device)
    # the flat [world * rows, words] view is the form every backend accepts
    dist.all_gather_into_tensor(out.view(world * packets.shape[0], *packets.shape[1:]), packets.contiguous(), group=group)
    return out


class _IpcHandle(_ctypes.Structure):
    """cudaIpcMemHandle_t"""
    _fields_ = [("reserved", _ctypes.c_char * 64)]


class _RawCudaInts:
    """int32 view of raw device memory, for torch.as_tensor."""

    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<i4", "data": (ptr, False), "version": 2}


class PeerPacketExchange:
    """The packets of every rank, delivered by stores into peer memory over NVLink instead of an all-gather.

    Every rank owns a receive buffer (two steps deep) and a flag array; both are mapped into the other ranks'
    processes through CUDA IPC (the handles travel once, through the process group; every rank opens them with
    its own device current, so that its kernels may store into them).  A step is
    `push(packets)`: a kernel stores this rank's packets into every rank's buffer and raises its flag there;
    `gathered()` makes the stream wait (bounded) for the flags of all ranks and returns the [world, rows, words]
    view to merge.  `timed_out()` tells, after a synchronisation, whether a wait ever gave up."""

    def __init__(self, rows: int, words: int, group=None, device=None, max_polls: int = 1 << 20):
        import ctypes

        from . import capi

        self.capi, self.group = capi, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dev, self.rows, self.words, self.max_polls = dev, rows, words, max_polls
        # One plain cudaMalloc allocation per rank (its IPC handle names the whole allocation, so it must not be
        # a piece of a pooled block): the receive slots, then the flags.
        slot_words = 2 * self.world * rows * words
        self._flag_offset = ((slot_words * 4 + 255) // 256) * 256
        nbytes = self._flag_offset + 256 * ((2 * self.world * 4 + 255) // 256)
        self._rt = rt = ctypes.CDLL("libcudart.so.12")
        rt.cudaIpcOpenMemHandle.argtypes = [ctypes.POINTER(ctypes.c_void_p), _IpcHandle, ctypes.c_uint]
        rt.cudaMalloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t]
        rt.cudaMemset.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]
        rt.cudaIpcGetMemHandle.argtypes = [ctypes.POINTER(_IpcHandle), ctypes.c_void_p]
        rt.cudaFree.argtypes = [ctypes.c_void_p]
        base, handle = ctypes.c_void_p(), _IpcHandle()
        with torch.cuda.device(dev):
            self._cuda(rt.cudaMalloc(ctypes.byref(base), nbytes), "cudaMalloc")
            self._base = base.value
            self._cuda(rt.cudaMemset(base, 0, nbytes), "cudaMemset")
            self._cuda(rt.cudaIpcGetMemHandle(ctypes.byref(handle), base), "cudaIpcGetMemHandle")
        region = torch.as_tensor(_RawCudaInts(self._base, nbytes // 4), device=dev)
        self.slots = region[:slot_words].view(2, self.world, rows, words)
        self.flags = region[self._flag_offset // 4:self._flag_offset // 4 + 2 * self.world].view(2, self.world)
        self.tickets = torch.zeros(self.world, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, bytes(handle), group=group)
        # Every rank opens the peers' handles with ITS OWN device current and lazy peer access: that is what maps
        # a peer's memory for kernels of this device.
        self._peer_bases = []
        slot_ptrs, flag_ptrs = [], []
        for r, h in enumerate(everyone):
            if r == self.rank:
                pbase = self._base
            else:
                opened = ctypes.c_void_p()
                with torch.cuda.device(dev):
                    self._cuda(rt.cudaIpcOpenMemHandle(ctypes.byref(opened), _IpcHandle.from_buffer_copy(h), 1),
                               "cudaIpcOpenMemHandle")
                pbase = opened.value
                self._peer_bases.append(pbase)
            slot_ptrs.append(pbase)
            flag_ptrs.append(pbase + self._flag_offset)
        self.slot_ptrs = torch.tensor(slot_ptrs, dtype=torch.int64, device=dev)
        self.flag_ptrs = torch.tensor(flag_ptrs, dtype=torch.int64, device=dev)
        self.seq = 0
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)  # nobody pushes before every rank has mapped and zeroed its buffers

    @staticmethod
    def _cuda(rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUDA error {rc}")

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (call it on every rank, after a barrier)."""
        import ctypes

        if getattr(self, "_base", None):
            torch.cuda.synchronize(self.dev)
            self._rt.cudaIpcCloseMemHandle.argtypes = [ctypes.c_void_p]
            for pbase in self._peer_bases:
                self._rt.cudaIpcCloseMemHandle(ctypes.c_void_p(pbase))
            self._rt.cudaFree(ctypes.c_void_p(self._base))
            self._base = None

    def push(self, packets: torch.Tensor) -> None:
        self.seq += 1
        self.capi.packets_push(packets, self.slot_ptrs, self.flag_ptrs, self.rank, self.world, self.seq, self.tickets)

    def gathered(self) -> torch.Tensor:
        self.capi.packets_wait(self.flags, self.world, self.seq, self.status, self.max_polls)
        return self.slots[self.seq & 1]

    def timed_out(self) -> bool:
        return int(self.status.item()) != 0


class VocabShardedSoftmaxTopk:
    """Fused Softmax + TopK over logits whose columns are split across the ranks of a process group."""

    def __init__(self, rows: int, shard_cols: int, index_offset: int, k: int, dtype: torch.dtype,
                 inv_temperature: float = 1.0, index_dtype: int = 0, group=None, device=None, exchange: str = "nccl"):
        """exchange: "nccl" = all-gather of the packets through the process group; "peer" = stores into peer
        memory, orchestrated here (PeerPacketExchange; CUDA devices of one node); "native" = the same exchange
        owned by the C++ operator ops::SoftmaxTopkSharded (one call per step; this class only carries the IPC
        handles through the process group)."""
        from . import capi

        self.capi = capi
        self.rows, self.k, self.dtype, self.inv_t = rows, k, dtype, inv_temperature
        self.index_offset, self.index_dtype, self.group = index_offset, index_dtype, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        words = capi.packet_bytes(k) // 4
        self.packets = torch.empty((rows, words), dtype=torch.int32, device=dev)
        self.gathered = torch.empty((self.world, rows, words), dtype=torch.int32, device=dev)
        self.values = torch.empty((rows, k), dtype=dtype, device=dev)
        self.indices = torch.empty((rows, k), dtype=torch.int64 if index_dtype == capi.I64 else torch.int32, device=dev)
        desc = capi.SoftmaxTopkDesc(rows=rows, cols=shard_cols, row_stride=shard_cols, dtype=capi._TORCH_DTYPE[dtype], k=k,
                                    index_dtype=index_dtype, value_kind=capi.VALUE_PROBABILITY,
                                    inv_temperature=inv_temperature, largest=1, path=0, splits=0,
                                    index_offset=index_offset)
        self.workspace = capi.Workspace(capi.softmax_topk_workspace_bytes(desc), dev)
        self.peer = PeerPacketExchange(rows, words, group, dev) if (exchange == "peer" and self.world > 1) else None
        self.native = None
        if exchange == "native":
            from . import host_api

            rank = dist.get_rank(group) if self.world > 1 else 0
            self.native = host_api.ShardedRank(dev.index if dev.index is not None else torch.cuda.current_device(), rank,
                                               self.world, rows, shard_cols, index_offset, k, capi._TORCH_DTYPE[dtype],
                                               index_dtype, inv_temperature)
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, self.native.handle(), group=group)
                self.native.connect(handles)
                dist.barrier(group=group)  # nobody pushes before every rank has mapped its peers

    def timed_out(self) -> bool:
        """After a synchronisation: has a bounded wait for the peers' packets ever given up?"""
        if self.native is not None:
            return self.native.timed_out()
        return self.peer.timed_out() if self.peer is not None else False

    def close(self) -> None:
        """Unmaps the peers' buffers (call it on every rank, after a barrier)."""
        if self.native is not None:
            self.native.close()
            self.native = None
        if self.peer is not None:
            self.peer.close()

    def __call__(self, shard_logits: torch.Tensor):
        capi = self.capi
        if self.native is not None:
            self.native.run(shard_logits.data_ptr(), self.values.data_ptr(), self.indices.data_ptr(),
                            torch.cuda.current_stream(shard_logits.device).cuda_stream)
            return self.values, self.indices
        capi.softmax_topk_partial(shard_logits, self.k, self.index_offset, self.inv_t, workspace=self.workspace,
                                  packets=self.packets)
        if self.peer is not None:
            self.peer.push(self.packets)
            gathered = self.peer.gathered()
        elif self.world > 1:
            exchange_packets(self.packets, self.group, self.gathered)
            gathered = self.gathered
        else:
            gathered = self.packets.unsqueeze(0)
        return capi.softmax_topk_merge(gathered, self.rows, self.k, self.dtype, self.inv_t, self.index_dtype,
                                       out=(self.values, self.indices))
