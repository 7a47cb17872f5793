"""Dropless-MoE plumbing around the block-sparse products: the block-diagonal topology of a
batch of tokens routed to experts, the token permutation into padded expert order, and the
expert-parallel exchange between GPUs.

This is the caller's side of stk.Matrix / stk.ops.sdd / stk.ops.dsd in a dMoE layer.  The
reference has no such code (it is a matmul library); the shapes follow the benchmark
configurations: tokens of expert e occupy ceil(count_e / 128) block rows, and those block rows
have nonzero blocks exactly in expert e's ffn / 128 block columns.
"""
import torch
import torch.distributed as dist

from stk_b200.backend import kernels as _kernels
from stk_b200.matrix import Matrix

BLOCK = 128


def padded_bins(counts, block=BLOCK):
    """(padded counts, exclusive start of every expert's padded bin, total padded rows)."""
    padded = ((counts + block - 1) // block) * block
    starts = torch.cumsum(padded, 0) - padded
    return padded, starts, int(padded.sum().item())


def block_diagonal_topology(padded_counts, ffn, dtype, device, block=BLOCK, data=None):
    """stk.Matrix of shape [sum(padded), E*ffn] whose block row r (belonging to expert e) holds
    the ffn/block consecutive column blocks of expert e.  The transposed metadata comes from the
    library's transpose kernel, as for any user-built Matrix."""
    num_experts = padded_counts.numel()
    cols_per_expert = ffn // block
    # Counts that already live on the host (the exchange has them there) cost no device sync.
    block_rows = int((padded_counts // block).sum())
    rows_per_expert = (padded_counts // block).to(device, non_blocking=True)
    expert_of_row = torch.repeat_interleave(
        torch.arange(num_experts, device=device), rows_per_expert, output_size=block_rows)
    row_indices = torch.repeat_interleave(
        torch.arange(block_rows, device=device, dtype=torch.int16), cols_per_expert)
    column_indices = (expert_of_row[:, None] * cols_per_expert +
                      torch.arange(cols_per_expert, device=device)[None, :]).reshape(-1).to(torch.int16)
    offsets = (torch.arange(block_rows + 1, device=device) * cols_per_expert).to(torch.int32)
    nnz = block_rows * cols_per_expert
    if data is None:
        data = torch.empty((nnz, block, block), dtype=dtype, device=device)
    size = torch.Size((block_rows * block, num_experts * ffn))
    if cols_per_expert % 2 == 0:
        # Known by construction: all block rows of an expert share one column list, column pairs
        # never straddle experts; only row pairs at expert boundaries fail to pair.
        _kernels.set_pair_hints(column_indices, 0.9, 1.0, 0.9, True)
    return Matrix(size, data, row_indices, column_indices, offsets)


def route_top1(expert_ids, num_experts, block=BLOCK):
    """Permutation of tokens into padded expert order for top-1 routing.

    Returns (slot, padded, starts, total): token t goes to row slot[t] of the padded buffer;
    rows that no token maps to are padding and must be zero."""
    counts = torch.bincount(expert_ids, minlength=num_experts)
    padded, starts, total = padded_bins(counts, block)
    order = torch.argsort(expert_ids, stable=True)
    sorted_experts = expert_ids[order]
    rank_in_expert = torch.arange(expert_ids.numel(), device=expert_ids.device) - \
        (torch.cumsum(counts, 0) - counts)[sorted_experts]
    slot = torch.empty_like(order)
    slot[order] = starts[sorted_experts] + rank_in_expert
    return slot, padded, starts, total


def permute_tokens(x, slot, total_rows):
    """Padded, expert-ordered copy of the token matrix x [T, h] (padding rows are zero)."""
    out = torch.zeros((total_rows, x.shape[1]), dtype=x.dtype, device=x.device)
    out[slot] = x
    return out


def unpermute_tokens(y, slot):
    """Inverse of permute_tokens: row t of the result is row slot[t] of y."""
    return y[slot]


class ExpertParallelExchange:
    """Token exchange of an expert-parallel dMoE layer: rank g owns experts
    [g*E/n, (g+1)*E/n); every rank starts with its own tokens and their expert ids.

    dispatch(): tokens travel to the owner of their expert (all_to_all_single with per-rank
    split sizes, after the per-expert counts have been exchanged); the receiver places them by
    local expert, every expert padded to a multiple of 128 rows.  combine(): the results travel
    back and are put in the sender's original token order.  One host read-back per dispatch (the
    counts; NCCL needs the split sizes on the host).  Works with any torch.distributed backend
    (NCCL over NVLink on the GPUs, gloo on the host for tests).
    """

    def __init__(self, num_experts, group=None, block=BLOCK):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts = num_experts
        self.local_experts = num_experts // self.world
        self.block = block

    def dispatch(self, x, expert_ids):
        """Returns (x_padded [T'_local, h], padded_counts (host int64 [local_experts]), state)."""
        dev = x.device
        world, local = self.world, self.local_experts
        # Send order: by expert (hence by destination rank), stable in the token index.
        send_order = torch.argsort(expert_ids, stable=True)
        counts = torch.empty((2, self.num_experts), dtype=torch.int64, device=dev)
        counts[0] = torch.bincount(expert_ids, minlength=self.num_experts)
        # counts[0][e] for the experts of rank g go to rank g: one row of E/n counts per peer
        dist.all_to_all_single(counts[1], counts[0], group=self.group)
        host = counts.cpu()                                  # the one synchronisation
        send_splits = host[0].view(world, local).sum(1).tolist()
        recv_by_peer = host[1].view(world, local)            # [peer, local expert]
        recv_splits = recv_by_peer.sum(1).tolist()
        received = sum(recv_splits)
        recv = torch.empty((received, x.shape[1]), dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv, x.index_select(0, send_order), recv_splits, send_splits,
                               group=self.group)
        # Rows arrive ordered (peer, local expert) in world*local contiguous segments; segment
        # (peer, e) goes to bin e behind the segments of lower peers.  All bookkeeping on the host.
        per_expert = recv_by_peer.sum(0)
        padded = ((per_expert + self.block - 1) // self.block) * self.block
        bin_start = torch.cumsum(padded, 0) - padded
        seg_len = recv_by_peer.reshape(-1)
        src_start = torch.cumsum(seg_len, 0) - seg_len
        within = torch.cumsum(recv_by_peer, 0) - recv_by_peer          # rows of lower peers in bin e
        dst_start = (bin_start[None, :] + within).reshape(-1)
        shift = (dst_start - src_start).to(dev, non_blocking=True)
        slot = torch.arange(received, device=dev) + torch.repeat_interleave(
            shift, seg_len.to(dev, non_blocking=True), output_size=received)
        total = int(padded.sum())
        x_padded = permute_tokens(recv, slot, total)
        state = dict(send_order=send_order, send_splits=send_splits, recv_splits=recv_splits,
                     slot=slot, tokens=x.shape[0])
        return x_padded, padded, state

    def combine(self, y_padded, state):
        """Inverse of dispatch for the per-token results y_padded [T'_local, h_out]."""
        back = y_padded.index_select(0, state["slot"])
        out_sorted = torch.empty((state["tokens"], y_padded.shape[1]), dtype=y_padded.dtype,
                                 device=y_padded.device)
        dist.all_to_all_single(out_sorted, back, state["send_splits"], state["recv_splits"],
                               group=self.group)
        out = torch.empty_like(out_sorted)
        out[state["send_order"]] = out_sorted
        return out
