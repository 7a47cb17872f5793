"""Host-side tests of the dMoE plumbing, including the expert-parallel exchange on 2 gloo ranks."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def check_routing(dmoe, x, ids, experts):
    index, padded, bin_rows, total = dmoe.route_top1(ids, experts)
    assert total == int(padded.sum()) and bool((padded % 128 == 0).all())
    assert bin_rows.cpu().tolist() == (padded // 128).tolist()
    xp = dmoe.permute_tokens(x, index, total)
    assert torch.equal(dmoe.unpermute_tokens(xp, index, x.shape[0]), x)
    counts = torch.bincount(ids.cpu(), minlength=experts)
    starts = torch.cumsum(padded, 0) - padded
    for e in range(experts):
        rows = xp[starts[e]:starts[e] + padded[e]].cpu()
        assert torch.equal(rows[:counts[e]], x.cpu()[ids.cpu() == e])   # stable order inside an expert
        assert torch.count_nonzero(rows[counts[e]:]).item() == 0      # zero padding


def test_route_top1_and_padding():
    from stk_b200 import dmoe
    torch.manual_seed(0)
    check_routing(dmoe, torch.randn(1000, 8), torch.randint(0, 4, (1000,)), 4)
    check_routing(dmoe, torch.randn(300, 8), torch.randint(0, 2, (300,)) * 3, 5)   # empty experts


def _exchange_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from stk_b200 import dmoe
        torch.manual_seed(100 + rank)
        E, h, T = 6, 5, 300 + 17 * rank
        ids = torch.randint(0, E, (T,))
        x = torch.randn(T, h)
        ex = dmoe.ExpertParallelExchange(E)
        xp, bin_rows, state = ex.dispatch(x, ids)
        padded = bin_rows.long() * 128
        assert xp.shape[0] == int(padded.sum()) == state["block_rows"] * 128
        # every local expert's bin holds exactly the tokens routed to it from all ranks,
        # ordered by source rank then token index, then zero padding
        gathered = [None] * world
        dist.all_gather_object(gathered, (x, ids))
        starts = torch.cumsum(padded, 0) - padded
        for le in range(ex.local_experts):
            e = rank * ex.local_experts + le
            expect = torch.cat([gx[gi == e] for gx, gi in gathered])
            rows = xp[starts[le]:starts[le] + padded[le]]
            assert torch.equal(rows[:expect.shape[0]], expect)
            assert torch.count_nonzero(rows[expect.shape[0]:]).item() == 0
        # an "expert computation" that tags rows with the global expert id, then the way back
        tag = torch.repeat_interleave(torch.arange(ex.local_experts) + rank * ex.local_experts, padded)
        y = xp * 2 + tag[:, None].float() * (xp.abs().sum(1, keepdim=True) > 0)
        out = ex.combine(y, state)
        assert torch.allclose(out, x * 2 + ids[:, None].float())
        # mismatched expert count is a host-side error, raised before any collective
        try:
            dmoe.ExpertParallelExchange(7)
            raise AssertionError("expected ValueError")
        except ValueError:
            pass
        open(os.path.join(tmp, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_two_ranks(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_exchange_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")
