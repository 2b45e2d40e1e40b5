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


class VocabShardedSoftmaxTopk:
    """Fused Softmax + TopK over logits whose columns are split across the ranks of a process group."""

    def __init__(self, rows: int, shard_cols: int, index_offset: int, k: int, dtype: torch.dtype,
                 inv_temperature: float = 1.0, index_dtype: int = 0, group=None, device=None):
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
        probe = torch.empty((rows, shard_cols), dtype=dtype, device="meta")
        desc = capi.SoftmaxTopkDesc(rows=rows, cols=shard_cols, row_stride=shard_cols, dtype=capi._TORCH_DTYPE[dtype], k=k,
                                    index_dtype=index_dtype, value_kind=capi.VALUE_PROBABILITY,
                                    inv_temperature=inv_temperature, largest=1, path=0, splits=0,
                                    index_offset=index_offset)
        del probe
        self.workspace = capi.Workspace(capi.softmax_topk_workspace_bytes(desc), dev)

    def __call__(self, shard_logits: torch.Tensor):
        capi = self.capi
        capi.softmax_topk_partial(shard_logits, self.k, self.index_offset, self.inv_t, workspace=self.workspace,
                                  packets=self.packets)
        if self.world > 1:
            exchange_packets(self.packets, self.group, self.gathered)
            gathered = self.gathered
        else:
            gathered = self.packets.unsqueeze(0)
        return capi.softmax_topk_merge(gathered, self.rows, self.k, self.dtype, self.inv_t, self.index_dtype,
                                       out=(self.values, self.indices))
