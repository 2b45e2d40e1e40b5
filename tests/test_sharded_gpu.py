"""Vocabulary-sharded Softmax + TopK on two or more GPUs: one process per GPU; the packets travel either
through an NCCL all-gather or by stores into peer memory."""
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


def _worker(rank: int, world: int, port: int, q, exchange: str = "nccl"):
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
        op = VocabShardedSoftmaxTopk(64, hi - lo, lo, 64, x.dtype, exchange=exchange)
        v, i = op(shard)
        v, i = v.clone(), i.clone()
        v2, i2 = op(shard)  # scratch is reusable
        v2, i2 = v2.clone(), i2.clone()
        # other logits in between and many steps back to back: the receive buffers are two steps deep
        y = workloads.sharded_vocab(rows=64, cols=256000, seed=77)
        yshard = y[:, lo:hi].contiguous().cuda()
        for _ in range(9):
            op(yshard)
            op(shard)
        vy, iy = op(yshard)
        torch.cuda.synchronize()
        wv, wi = util.oracle_softmax_topk(x, 64)
        wvy, wiy = util.oracle_softmax_topk(y, 64)
        ok = True
        try:
            util.assert_indices_equal(i, wi, f"rank {rank}")
            util.assert_probs_close(v, wv, x.dtype, f"rank {rank}")
            assert torch.equal(i, i2) and torch.equal(v, v2)
            util.assert_indices_equal(iy, wiy, f"rank {rank}, second input")
            util.assert_probs_close(vy, wvy, x.dtype, f"rank {rank}, second input")
            assert not op.timed_out()
        except AssertionError as e:
            ok = str(e)
        q.put((rank, ok))
        if op.peer is not None or op.native is not None:
            dist.barrier()  # no rank unmaps while another may still store into its memory
            op.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "peer", "native"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_vocab_sharded(world, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(r[1] is True for r in results), results


def test_packet_wait_gives_up_with_a_status():
    """A flag that nobody sets: the bounded wait returns VKOP_TIMEOUT in the status word and the context
    stays usable (no trap, no hang)."""
    from vkop_b200 import capi

    flags = torch.zeros((2, 4), dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.packets_wait(flags, 4, 1, status, max_polls=2000)
    torch.cuda.synchronize()
    assert int(status.item()) == -5
    # flags that are set let it through
    flags[1, :] = 3
    status.zero_()
    capi.packets_wait(flags, 4, 3, status, max_polls=2000)
    x = torch.randn(4, 1000, device="cuda")
    v, i = capi.softmax_topk(x, 5)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and i.shape == (4, 5)


def test_peer_exchange_kernels_with_emulated_ranks():
    """The push / wait / merge sequence of four ranks, emulated in one process on one GPU: every "rank" has its
    own receive buffer and flags, the pointer tables name all of them, and the kernels of the ranks run one
    after the other on one stream (so no kernel ever waits for a kernel that has not run)."""
    import oracle
    from tests import util
    from vkop_b200 import capi, workloads
    from vkop_b200.sharded import split_even

    world, rows, k = 4, 48, 64
    words = capi.packet_bytes(k) // 4
    dev = torch.device("cuda")
    slots = [torch.zeros((2, world, rows, words), dtype=torch.int32, device=dev) for _ in range(world)]
    flags = [torch.zeros((2, world), dtype=torch.int32, device=dev) for _ in range(world)]
    tickets = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    slot_ptrs = torch.tensor([t.data_ptr() for t in slots], dtype=torch.int64, device=dev)
    flag_ptrs = torch.tensor([t.data_ptr() for t in flags], dtype=torch.int64, device=dev)
    for seq in range(1, 6):
        x = workloads.sharded_vocab(rows=rows, cols=100000, seed=seq)
        for r in range(world):
            lo, hi = split_even(x.shape[1], world, r)
            packets = capi.softmax_topk_partial(x[:, lo:hi].contiguous().cuda(), k, lo)
            capi.packets_push(packets, slot_ptrs, flag_ptrs, r, world, seq, tickets[r])
        wv, wi = util.oracle_softmax_topk(x, k)
        for r in range(world):
            capi.packets_wait(flags[r], world, seq, status, max_polls=1000)
            v, i = capi.softmax_topk_merge(slots[r][seq & 1], rows, k, x.dtype)
            util.assert_indices_equal(i, wi, f"emulated rank {r}, step {seq}")
            util.assert_probs_close(v, wv, x.dtype, f"emulated rank {r}, step {seq}")
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_all_ranks_exchange_in_one_launch():
    """Four ranks on one GPU with their pushes and waits running CONCURRENTLY: one cooperative launch in which
    every rank's blocks store its packets into all receive buffers and raise the flags while the ranks'
    waiting blocks already poll theirs (the release / acquire pairing of the real exchange; separate
    launches that wait for one another are not allowed on one GPU).  512 rows, the row count of the
    vocabulary-sharded configuration; results of every rank against the oracle, over several steps; the
    bounded waits must not run out."""
    from tests import util
    from vkop_b200 import capi, workloads
    from vkop_b200.sharded import split_even

    world, rows, k = 4, 512, 64
    words = capi.packet_bytes(k) // 4
    dev = torch.device("cuda")
    slots = [torch.zeros((2, world, rows, words), dtype=torch.int32, device=dev) for _ in range(world)]
    flags = [torch.zeros((2, world), dtype=torch.int32, device=dev) for _ in range(world)]
    tickets = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(world, dtype=torch.int32, device=dev)
    packets = [torch.empty((rows, words), dtype=torch.int32, device=dev) for _ in range(world)]
    ptr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    slot_ptrs, flag_ptrs, ticket_ptrs, packet_ptrs = ptr(slots), ptr(flags), ptr(tickets), ptr(packets)
    for seq in range(1, 5):
        x = workloads.sharded_vocab(rows=rows, cols=64000, seed=40 + seq)
        xg = x.cuda()
        for r in range(world):
            lo, hi = split_even(x.shape[1], world, r)
            capi.softmax_topk_partial(xg[:, lo:hi].contiguous(), k, lo, packets=packets[r])
        capi.packets_exchange_all_ranks(packet_ptrs, rows * words * 4, slot_ptrs, flag_ptrs, world, seq, ticket_ptrs, status,
                                        max_polls=200000)
        wv, wi = util.oracle_softmax_topk(x, k)
        for r in range(world):
            v, i = capi.softmax_topk_merge(slots[r][seq & 1], rows, k, x.dtype)
            util.assert_indices_equal(i, wi, f"rank {r}, step {seq}")
            util.assert_probs_close(v, wv, x.dtype, f"rank {r}, step {seq}")
        assert status.cpu().tolist() == [0] * world, "a bounded wait ran out"


def test_native_sharded_operator_on_one_gpu():
    """ops::SoftmaxTopkSharded through its flat C entry points.  One rank: partial + merge.  Two ranks living in one
    process on one GPU (connect_local): both begin (partial + push), then both finish (wait + merge), all on one
    stream, so that no kernel ever waits for one that is enqueued behind it."""
    import oracle  # noqa: F401
    from tests import util
    from vkop_b200 import capi, host_api, workloads
    from vkop_b200.sharded import split_even

    rows, cols, k = 48, 131072, 64
    x = workloads.sharded_vocab(rows=rows, cols=cols)
    xg = x.cuda()
    wv, wi = util.oracle_softmax_topk(x, k)
    dt = capi._TORCH_DTYPE[x.dtype]
    stream = torch.cuda.current_stream().cuda_stream
    # one rank holds every column
    one = host_api.ShardedRank(0, 0, 1, rows, cols, 0, k, dt)
    v = torch.empty((rows, k), dtype=x.dtype, device="cuda")
    i = torch.empty((rows, k), dtype=torch.int32, device="cuda")
    one.run(xg.data_ptr(), v.data_ptr(), i.data_ptr(), stream)
    torch.cuda.synchronize()
    util.assert_indices_equal(i, wi, "one rank")
    util.assert_probs_close(v, wv, x.dtype, "one rank")
    one.close()
    # three ranks of this process
    world = 3
    shards, ranks, outs = [], [], []
    for r in range(world):
        lo, hi = split_even(cols, world, r)
        shards.append(xg[:, lo:hi].contiguous())
        ranks.append(host_api.ShardedRank(0, r, world, rows, hi - lo, lo, k, dt, capi.I64))
        outs.append((torch.zeros((rows, k), dtype=x.dtype, device="cuda"), torch.zeros((rows, k), dtype=torch.int64, device="cuda")))
    for r in ranks:
        r.connect_local(ranks)
    y = workloads.sharded_vocab(rows=rows, cols=cols, seed=5)
    yshards = [y.cuda()[:, split_even(cols, world, r)[0]:split_even(cols, world, r)[1]].contiguous() for r in range(world)]
    for step in range(7):  # the receive slots are two steps deep: many steps, alternating inputs
        src = shards if step % 2 == 0 else yshards
        for r in range(world):
            ranks[r].begin(src[r].data_ptr(), stream)
        for r in range(world):
            ranks[r].finish(outs[r][0].data_ptr(), outs[r][1].data_ptr(), stream)
    torch.cuda.synchronize()
    for r in range(world):
        assert not ranks[r].timed_out()
        util.assert_indices_equal(outs[r][1], wi, f"rank {r} of {world}")
        util.assert_probs_close(outs[r][0], wv, x.dtype, f"rank {r} of {world}")
    for r in ranks:
        r.close()
