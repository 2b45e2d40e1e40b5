"""Vocabulary-sharded Softmax + TopK on two or more GPUs (NCCL): one process per GPU."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    import torch.distributed as dist

    import oracle
    from tests import util
    from vkop_b200 import workloads
    from vkop_b200.sharded import VocabShardedSoftmaxTopk, split_even

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        x = workloads.sharded_vocab(rows=64, cols=256000)
        lo, hi = split_even(x.shape[1], world, rank)
        shard = x[:, lo:hi].contiguous().cuda()
        op = VocabShardedSoftmaxTopk(64, hi - lo, lo, 64, x.dtype)
        v, i = op(shard)
        v2, i2 = op(shard)  # scratch is reusable
        torch.cuda.synchronize()
        wv, wi = util.oracle_softmax_topk(x, 64)
        ok = True
        try:
            util.assert_indices_equal(i, wi, f"rank {rank}")
            util.assert_probs_close(v, wv, x.dtype, f"rank {rank}")
            assert torch.equal(i, i2) and torch.equal(v, v2)
        except AssertionError as e:
            ok = str(e)
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_vocab_sharded_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(r[1] is True for r in results), results
