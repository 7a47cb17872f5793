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


def check_topk(dmoe, x, ids, weights, experts, tol=1e-5):
    """Top-k routing: every (token, choice) slot lands in its expert's bin, and the weighted combine
    of per-slot results gives sum_j w[t, j] * f(x[t])."""
    tokens, k = ids.shape
    index, position, padded, bin_rows, total = dmoe.route_topk(ids, experts)
    assert total == int(padded.sum()) and index.numel() == total and position.numel() == tokens * k
    xp = dmoe.permute_tokens(x, index, total, top_k=k)
    idx, pos = index.cpu().long(), position.cpu().long()
    assert torch.equal(idx[pos], torch.arange(tokens * k))               # position inverts index
    flat = ids.cpu().reshape(-1)
    starts = torch.cumsum(padded, 0) - padded
    for e in range(experts):
        rows = xp[starts[e]:starts[e] + padded[e]].cpu()
        slots = torch.nonzero(flat == e).view(-1)
        assert torch.equal(rows[:slots.numel()], x.cpu()[slots // k])    # stable slot order inside an expert
        assert torch.count_nonzero(rows[slots.numel():]).item() == 0
    out = dmoe.combine_tokens(xp * 2, position, weights, tokens, k)
    expect = 2 * x.float() * weights.float().sum(1, keepdim=True)
    assert torch.allclose(out.float().cpu(), expect.cpu(), rtol=tol, atol=tol)


def test_route_topk_and_weighted_combine():
    from stk_b200 import dmoe
    torch.manual_seed(1)
    check_topk(dmoe, torch.randn(500, 8), torch.randint(0, 6, (500, 2)), torch.rand(500, 2), 6)
    check_topk(dmoe, torch.randn(77, 8), torch.randint(0, 3, (77, 3)) * 2, torch.rand(77, 3), 7)


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
        # top-2 routing with weights through the same exchange
        ids2 = torch.randint(0, E, (T, 2))
        w2 = torch.rand(T, 2)
        xp2, bins2, st2 = ex.dispatch(x, ids2)
        assert xp2.shape[0] == int(bins2.sum()) * 128
        gathered = [None] * world
        dist.all_gather_object(gathered, (x, ids2))
        starts2 = torch.cumsum(bins2.long() * 128, 0) - bins2.long() * 128
        for le in range(ex.local_experts):
            e = rank * ex.local_experts + le
            expect = torch.cat([gx[torch.nonzero(gi.reshape(-1) == e).view(-1) // 2] for gx, gi in gathered])
            assert torch.equal(xp2[starts2[le]:starts2[le] + expect.shape[0]], expect)
        out2 = ex.combine(xp2 * 3, st2, w2)
        assert torch.allclose(out2, 3 * x * w2.sum(1, keepdim=True), rtol=1e-5, atol=1e-5)
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


def test_binding_the_host_side_to_a_gpu_changes_nothing_without_one():
    """No CUDA device, no NVML: the call reports 0 cores kept and leaves the process's affinity alone."""
    import os
    from stk_b200 import dmoe
    before = os.sched_getaffinity(0)
    assert dmoe.bind_host_to_gpu_node("cuda:0") == 0 or torch.cuda.is_available()
    if not torch.cuda.is_available():
        assert os.sched_getaffinity(0) == before
