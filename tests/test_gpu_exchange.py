"""Expert-parallel exchange over peer memory (stk_b200.dmoe.PeerExchange).

The kernels only see device pointers, so several ranks can be run inside one process on one GPU by
handing every emulated rank the others' buffers as its "peers": that covers the placement
arithmetic, the padding and the round trip bit-exactly.  With two GPUs the real thing (torch
symmetric memory, one process per GPU) is compared row for row with the NCCL exchange.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _emulated(world, experts, tokens_per_rank, hidden, capacity_rows, dtype=torch.float16, seed=0):
    from stk_b200 import dmoe
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    counts = [torch.zeros(world, experts, dtype=torch.int32, device=dev) for _ in range(world)]
    # 64 guard rows behind every receive buffer: nothing may ever be written there
    recv = [torch.full((capacity_rows + 64, hidden), float("nan"), dtype=dtype, device=dev)[:capacity_rows]
            for _ in range(world)]
    result = [torch.empty((capacity_rows, hidden), dtype=dtype, device=dev) for _ in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    peer_counts, peer_recv, peer_result = ptrs(counts), ptrs(recv), ptrs(result)
    ranks = []
    for r in range(world):
        buffers = dmoe.PeerExchangeBuffers(counts[r], recv[r], result[r], peer_counts, peer_recv, peer_result)
        ex = dmoe.PeerExchange(experts, tokens_per_rank[r], hidden, hidden, dtype, dev, world=world, rank=r,
                               capacity_rows=capacity_rows, buffers=buffers, barrier=lambda channel: None)
        x = torch.randn(tokens_per_rank[r], hidden, generator=g).to(dtype).to(dev)
        ids = torch.randint(0, experts, (tokens_per_rank[r],), generator=g).to(torch.int32)
        ids[ids == 3] = 2                                  # an expert nobody routes to
        ranks.append((ex, x, ids.to(dev)))
    return ranks, recv


@pytest.mark.parametrize("world,tokens", [(2, [700, 450]), (4, [300, 0, 513, 129])])
def test_emulated_ranks_round_trip(world, tokens):
    from stk_b200.backend import lib
    experts, hidden, block = 8, 64, 128
    ranks, recv = _emulated(world, experts, tokens, hidden, capacity_rows=4096)
    local = experts // world
    sorted_ = [ex.share_counts(ids) for ex, _, ids in ranks]
    pushed = [ex.push(x, *so) for (ex, x, _), so in zip(ranks, sorted_)]
    totals = [ex.padded_rows() for ex, _, _ in ranks]
    for d, (ex, _, _) in enumerate(ranks):
        # expected bins of rank d: expert by expert, source rank by source rank, original token order
        rows, bins = [], []
        for le in range(local):
            e = d * local + le
            part = [x[ids == e] for _, x, ids in ranks]
            n = sum(p.shape[0] for p in part)
            pad = (n + block - 1) // block * block - n
            rows += part + [torch.zeros(pad, hidden, dtype=part[0].dtype, device=part[0].device)]
            bins.append((n + pad) // block)
        expected = torch.cat(rows)
        assert totals[d] == expected.shape[0]
        assert torch.equal(recv[d][:totals[d]].view(torch.int16), expected.view(torch.int16))
        assert pushed[d][1].tolist() == bins
    states = []
    for (ex, x, _), (dest, _), total in zip(ranks, pushed, totals):
        state = dict(dest=dest, tokens=x.shape[0], total=total, block_rows=total // block)
        ex.publish(ex.buf.recv[:total] * 2, state)
        states.append(state)
    for (ex, x, _), state in zip(ranks, states):
        out = ex.pull(state)
        assert torch.equal(out, x * 2)
    assert lib.device_status() == 0


def test_capacity_overflow_is_reported_not_written():
    from stk_b200.backend import lib
    ranks, recv = _emulated(2, 8, [600, 600], 64, capacity_rows=256)
    sorted_ = [ex.share_counts(ids) for ex, _, ids in ranks]
    for (ex, x, _), so in zip(ranks, sorted_):
        ex.push(x, *so)
    with pytest.raises(RuntimeError, match="capacity_rows"):
        ranks[0][0].padded_rows()
    assert lib.device_status() == -7                       # STK_ERR_WORKSPACE, recorded by the kernel
    assert lib.device_status() == 0                        # reading clears it
    for r in recv:
        guard = torch.as_strided(r, (64, r.shape[1]), r.stride(), r.shape[0] * r.shape[1])
        assert bool(torch.isnan(guard).all())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank, world, port, result_queue):
    import torch.distributed as dist
    from stk_b200 import dmoe
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        experts, tokens, hidden = 8, 3000 + 17 * rank, 256
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(tokens, hidden, generator=g).half().to(dev)
        ids = torch.randint(0, experts, (tokens,), generator=g).to(torch.int32).to(dev)
        ref = dmoe.ExpertParallelExchange(experts)
        peer = dmoe.PeerExchange(experts, tokens, hidden, hidden, torch.float16, dev)
        ok = True
        for _ in range(3):                                  # the buffers are reused from step to step
            xp_ref, bins_ref, st_ref = ref.dispatch(x, ids)
            xp, bins, st = peer.dispatch(x, ids)
            ok &= torch.equal(xp, xp_ref) and torch.equal(bins, bins_ref)
            ok &= torch.equal(peer.combine(xp * 3, st), ref.combine(xp_ref * 3, st_ref))
            x = x + 1
        torch.cuda.synchronize()
        result_queue.put((rank, bool(ok)))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_peer_exchange_matches_nccl():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_two_gpu_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs)
    results = dict(queue.get(timeout=10) for _ in range(2))
    assert results == {0: True, 1: True}
