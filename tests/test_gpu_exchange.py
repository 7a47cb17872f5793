"""Expert-parallel exchange over peer memory (stk_b200.dmoe.PeerExchange), top-1 and top-2 routing.

The kernels only see device pointers, so several ranks can be run inside one process on one GPU by
handing every emulated rank the others' buffers as its "peers" (the barrier becomes a no-op, the
phases are run rank by rank): that covers the placement arithmetic, the padding, the tags, the
chunked push and the weighted way back bit-exactly.  With two GPUs the real thing (torch symmetric
memory, one process per GPU, the library's barrier kernel) is compared with the NCCL exchange.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _emulated(world, experts, tokens_per_rank, hidden, capacity_rows, top_k=1, chunks=1, dtype=torch.float16,
              seed=0):
    from stk_b200 import dmoe
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    slot_rows = max(tokens_per_rank) * top_k
    counts = [torch.zeros(world, experts, dtype=torch.int32, device=dev) for _ in range(world)]
    # 64 guard rows behind every receive buffer: nothing may ever be written there
    recv = [torch.full((capacity_rows + 64, hidden), float("nan"), dtype=dtype, device=dev)[:capacity_rows]
            for _ in range(world)]
    tags = [torch.full((capacity_rows,), -7, dtype=torch.int64, device=dev) for _ in range(world)]
    slots = [torch.full((slot_rows, hidden), float("nan"), dtype=dtype, device=dev) for _ in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    shared = (ptrs(counts), ptrs(recv), ptrs(tags), ptrs(slots))
    ranks = []
    for r in range(world):
        buffers = dmoe.PeerExchangeBuffers(counts[r], recv[r], tags[r], slots[r], *shared)
        ex = dmoe.PeerExchange(experts, tokens_per_rank[r], hidden, hidden, dtype, dev, world=world, rank=r,
                               capacity_rows=capacity_rows, buffers=buffers, barrier=lambda channel: None,
                               top_k=top_k, chunks=chunks)
        ex.slot_rows = slot_rows
        x = torch.randn(tokens_per_rank[r], hidden, generator=g).to(dtype).to(dev)
        shape = (tokens_per_rank[r],) if top_k == 1 else (tokens_per_rank[r], top_k)
        ids = torch.randint(0, experts, shape, generator=g).to(torch.int32)
        ids[ids == 3] = 2                                  # an expert nobody routes to
        w = torch.rand(tokens_per_rank[r], top_k, generator=g).to(dev)
        ranks.append((ex, x, ids.to(dev), w))
    return ranks, recv


@pytest.mark.parametrize("world,tokens,top_k,chunks", [(2, [700, 450], 1, 1), (4, [300, 0, 513, 129], 1, 1),
                                                        (2, [700, 450], 2, 2), (4, [300, 0, 513, 129], 2, 2),
                                                        (2, [257, 640], 2, 4)])
def test_emulated_ranks_round_trip(world, tokens, top_k, chunks):
    from stk_b200.backend import lib
    experts, hidden, block = 8, 64, 128
    ranks, recv = _emulated(world, experts, tokens, hidden, capacity_rows=4096, top_k=top_k, chunks=chunks)
    local = experts // world
    sorted_ = [ex.share_counts(ids) for ex, _, ids, _ in ranks]
    plans = [ex.plan() for ex, _, _, _ in ranks]
    for c in range(chunks):                               # all ranks push chunk c, then chunk c + 1
        for (ex, x, _, _), so, (dest_base, _) in zip(ranks, sorted_, plans):
            ex.push(x, *so, dest_base, c, chunks)
    totals = [ex.totals() for ex, _, _, _ in ranks]
    for d, (ex, _, _, _) in enumerate(ranks):
        # expected bins of rank d: expert by expert, source rank by source rank, slot order
        rows, bins, per_chunk = [], [], [0] * chunks
        for le in range(local):
            e = d * local + le
            part = []
            for _, x, ids, _ in ranks:
                flat = ids.reshape(-1)
                part.append(x[torch.nonzero(flat == e).view(-1) // top_k])
            n = sum(p.shape[0] for p in part)
            pad = (n + block - 1) // block * block - n
            rows += part + [torch.zeros(pad, hidden, dtype=part[0].dtype, device=part[0].device)]
            bins.append((n + pad) // block)
            per_chunk[le * chunks // local] += n + pad
        expected = torch.cat(rows)
        assert totals[d][0] == expected.shape[0]
        assert totals[d][2] == max(t[0] for t in totals)
        assert totals[d][3:] == per_chunk
        assert torch.equal(recv[d][:totals[d][0]].view(torch.int16), expected.view(torch.int16))
        assert plans[d][1].tolist() == bins
    # the "experts" double every row; results travel home chunk by chunk and are combined with weights
    for (ex, _, _, _), t in zip(ranks, totals):
        ex.result[:t[0]] = ex.buf.recv[:t[0]] * 2
    for c in range(chunks):
        for (ex, _, _, _), t in zip(ranks, totals):
            ex.give_back(sum(t[3:3 + c]), t[3 + c])
    for ex, x, _, w in ranks:
        out = ex.gather_slots(x.shape[0], w if top_k > 1 else None)
        expect = (2 * x).float() * (w.sum(1, keepdim=True) if top_k > 1 else 1.0)
        if top_k == 1:
            assert torch.equal(out, x * 2)
        else:
            assert torch.allclose(out.float(), expect, rtol=2e-3, atol=2e-3)
    assert lib.device_status() == 0


def test_capacity_overflow_is_reported_on_every_rank_and_nothing_is_written():
    from stk_b200.backend import lib
    ranks, recv = _emulated(2, 8, [900, 300], 64, capacity_rows=512)
    sorted_ = [ex.share_counts(ids) for ex, _, ids, _ in ranks]
    plans = [ex.plan() for ex, _, _, _ in ranks]
    for (ex, x, _, _), so, (dest_base, _) in zip(ranks, sorted_, plans):
        ex.push(x, *so, dest_base)
    for ex, _, _, _ in ranks:                              # the same decision on every rank
        with pytest.raises(RuntimeError, match="capacity_rows"):
            ex.totals()
    assert lib.device_status() == -7                       # STK_ERR_WORKSPACE, recorded by the kernel
    assert lib.device_status() == 0                        # reading clears it
    for r in recv:
        guard = torch.as_strided(r, (64, r.shape[1]), r.stride(), r.shape[0] * r.shape[1])
        assert bool(torch.isnan(guard).all())


def test_barrier_wait_is_bounded():
    """A barrier whose peer never signals gives up after its time limit and reports it through the
    status word; the context stays usable (nothing traps, nothing spins on)."""
    from stk_b200.backend import lib
    dev = torch.device("cuda", 0)
    flags = [torch.zeros(64, dtype=torch.int64, device=dev) for _ in range(2)]
    peer_flags = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    L = lib.load()
    lib.check(L.stk_b200_ep_barrier(lib.ptr(peer_flags), 2, 0, 1, 200, lib.stream_ptr(dev)), "stk_b200_ep_barrier")
    torch.cuda.synchronize()
    assert lib.device_status() == -10                      # STK_ERR_DEVICE_TIMEOUT
    assert flags[0][0].item() == 1 and flags[1][0].item() == 1   # this rank did signal both arrays
    # once the "peer" has signalled, the same barrier passes at once
    flags[0][1] = 1
    lib.check(L.stk_b200_ep_barrier(lib.ptr(peer_flags), 2, 0, 1, 200, lib.stream_ptr(dev)), "stk_b200_ep_barrier")
    torch.cuda.synchronize()
    assert lib.device_status() == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_worker(rank, world, port, result_queue):
    import torch.distributed as dist
    from stk_b200 import dmoe
    from stk_b200.backend import lib
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        experts, tokens, hidden, top_k = 8, 3000 + 17 * rank, 256, 2
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(tokens, hidden, generator=g).half().to(dev)
        ids = torch.randint(0, experts, (tokens, top_k), generator=g).to(torch.int32).to(dev)
        w = torch.rand(tokens, top_k, generator=g).to(dev)
        ref = dmoe.ExpertParallelExchange(experts)
        peer = dmoe.PeerExchange(experts, tokens, hidden, hidden, torch.float16, dev, top_k=top_k)
        chunked = dmoe.PeerExchange(experts, tokens, hidden, hidden, torch.float16, dev, top_k=top_k, chunks=2)
        ok = True
        for _ in range(3):                                  # the buffers are reused from step to step
            xp_ref, bins_ref, st_ref = ref.dispatch(x, ids)
            xp, bins, st = peer.dispatch(x, ids)
            ok &= torch.equal(xp, xp_ref) and torch.equal(bins, bins_ref)
            want = ref.combine(xp_ref * 3, st_ref, w)
            ok &= torch.equal(peer.combine(xp * 3, st, w), want)

            def triple(chunk, rows, bin_rows, block_rows, out):
                assert rows.shape[0] == block_rows * 128 == int(bin_rows.sum()) * 128
                torch.mul(rows, 3, out=out)
            ok &= torch.equal(chunked.forward(x, ids, w, triple), want)

            # with a prepare step: what it returns for a chunk (made on another stream, from the bin
            # sizes alone) reaches that chunk's expert function
            def scale_for(chunk, bin_rows, block_rows):
                return torch.full((1,), 3.0, dtype=torch.float16, device=dev), int(bin_rows.sum())

            def scaled(chunk, rows, bin_rows, block_rows, out, prepared):
                factor, blocks = prepared
                assert blocks == block_rows
                torch.mul(rows, factor, out=out)
            ok &= torch.equal(chunked.forward(x, ids, w, scaled, prepare_fn=scale_for), want)
            x = x + 1
        torch.cuda.synchronize()
        ok &= lib.device_status() == 0
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
