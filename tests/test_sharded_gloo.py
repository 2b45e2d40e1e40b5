"""World-size-2 CPU (gloo) test of the multi-GPU host logic: partitioning, the packet exchange and the merge
arithmetic.  The per-shard reduction and the merge run through the oracle here (no GPU); the CUDA kernels that
produce and consume the same packets are covered by the GPU tests."""
from __future__ import annotations

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tests import util
from vkop_b200 import workloads
from vkop_b200.sharded import exchange_packets, split_even

K = 16


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def pack(m, s, keys, idx, cnt, k):
    """Packet words as the library lays them out: m, s (float bits), count, 0, k keys, k indices."""
    rows = m.shape[0]
    out = np.zeros((rows, 4 + 2 * k), np.uint32)
    out[:, 0] = m.view(np.uint32)
    out[:, 1] = s.astype(np.float32).view(np.uint32)
    out[:, 2] = cnt.astype(np.uint32)
    out[:, 4:4 + k] = keys
    out[:, 4 + k:] = np.where(idx >= 0, idx, 0).astype(np.uint32)
    return torch.from_numpy(out.view(np.int32))


def unpack(words: np.ndarray, k):
    w = words.view(np.uint32)
    return (w[:, 0].copy().view(np.float32), w[:, 1].copy().view(np.float32).astype(np.float64), w[:, 4:4 + k],
            w[:, 4 + k:].astype(np.int64), w[:, 2].astype(np.int32))


def _worker(rank: int, world: int, port: int, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = workloads.sharded_vocab(rows=8, cols=5001)  # odd width: uneven slices
        xa = util.to_oracle_array(x)
        # --- vocabulary sharding ---
        lo, hi = split_even(x.shape[1], world, rank)
        mine = pack(*oracle.shard_packet(np.ascontiguousarray(xa[:, lo:hi]), K, lo, dtype=oracle.BF16), K)
        gathered = exchange_packets(mine)
        assert tuple(gathered.shape) == (world, 8, 4 + 2 * K)
        packets = [unpack(gathered[g].numpy(), K) for g in range(world)]
        v, i = util.merge_packets_reference(packets, K, xa, oracle.BF16)
        wv, wi = oracle.softmax_topk(xa, K, dtype=oracle.BF16)
        ok_vocab = bool(np.array_equal(i, wi) and np.all(np.abs(v - wv) <= 1e-6 + 1e-4 * np.abs(wv)))
        # --- row sharding: no exchange on the data path; results gathered only to compare ---
        r0, r1 = split_even(x.shape[0], world, rank)
        lv, li = oracle.softmax_topk(np.ascontiguousarray(xa[r0:r1]), K, dtype=oracle.BF16)
        parts = [None] * world
        dist.all_gather_object(parts, (r0, r1, li))
        full = np.concatenate([p[2] for p in sorted(parts, key=lambda p: p[0])])
        ok_rows = bool(np.array_equal(full, wi))
        q.put((rank, ok_vocab, ok_rows))
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] and r[2] for r in results), results
