"""Dropless-MoE plumbing around the block-sparse products: sorting tokens by expert, moving token
rows into and out of padded expert bins, the block-diagonal topology of a routed batch, and the
expert-parallel exchange between GPUs.

This is the caller's side of stk.Matrix / stk.ops.sdd / stk.ops.dsd in a dMoE layer.  The
reference has no such code (it is a matmul library); the shapes follow the benchmark
configurations: tokens of expert e occupy ceil(count_e / 128) block rows, and those block rows
have nonzero blocks exactly in expert e's ffn / 128 block columns.

On CUDA tensors everything below runs as kernels of libstk_b200.so (stable counting sort, row
gather / scatter with 16-byte accesses, closed-form topology); there is one host read-back per
routed batch (the per-expert counts, which size the padded buffers and, across GPUs, the NCCL split
sizes).  Host tensors take plain torch indexing instead - that path exists for the gloo tests of
the multi-rank bookkeeping, not for production use.
"""
import torch
import torch.distributed as dist

from stk_b200.backend import kernels as _kernels
from stk_b200.backend import lib as _lib
from stk_b200.matrix import Matrix

BLOCK = 128


# ------------------------------------------------------------------------------ building blocks
def sort_by_expert(expert_ids, num_experts):
    """Stable sort of token (or slot) indices by expert: (order int32 [T], offsets int32 [E+1])."""
    if expert_ids.is_cuda:
        ids16 = expert_ids.to(torch.int16)
        _, offsets, order = _kernels.transpose_meta(ids16, ids16, num_experts)
        return order, offsets
    order = torch.argsort(expert_ids, stable=True).to(torch.int32)
    counts = torch.bincount(expert_ids, minlength=num_experts)
    offsets = torch.cat([counts.new_zeros(1), torch.cumsum(counts, 0)]).to(torch.int32)
    return order, offsets


def gather_rows(src, index, n_out=None, index_div=1):
    """out[i] = src[index[i] // index_div], or a zero row where index[i] < 0.  index_div = k when
    `index` holds top-k slots (slot = token * k + choice) and `src` one row per token."""
    n_out = index.numel() if n_out is None else n_out
    if src.is_cuda:
        src = src.contiguous()
        out = torch.empty((n_out, src.shape[1]), dtype=src.dtype, device=src.device)
        with _lib.on_device(src.device):
            rc = _lib.load().stk_b200_gather_rows(
                _lib.ptr(src), _lib.ptr(out), _lib.ptr(index), n_out,
                src.shape[1] * src.element_size(), index_div, _lib.stream_ptr(src.device))
        _lib.check(rc, "stk_b200_gather_rows")
        return out
    out = src.new_zeros((n_out, src.shape[1]))
    valid = index >= 0
    out[valid] = src[torch.div(index[valid].long(), index_div, rounding_mode="floor")]
    return out


def weighted_sum_rows(src, position, weights, tokens, top_k):
    """out[t] = sum_j weights[t, j] * src[position[t*k + j]] (fp32 accumulation, one rounding): the
    top-k combine.  position None: src is slot-ordered; weights None: all ones (float32 [T, k] or
    [T*k] otherwise); a negative position contributes nothing."""
    if src.is_cuda:
        src = src.contiguous()
        out = torch.empty((tokens, src.shape[1]), dtype=src.dtype, device=src.device)
        if weights is not None:
            weights = weights.to(torch.float32).contiguous()
        with _lib.on_device(src.device):
            rc = _lib.load().stk_b200_weighted_sum_rows(
                _lib.ptr(src), _lib.ptr(position), _lib.ptr(weights), _lib.ptr(out), tokens, top_k,
                src.shape[1] * src.element_size(), _lib.dtype_code(src.dtype), _lib.stream_ptr(src.device))
        _lib.check(rc, "stk_b200_weighted_sum_rows")
        return out
    slots = tokens * top_k
    pos = torch.arange(slots) if position is None else position.long()
    rows = src.float()[pos.clamp(min=0)] * (pos >= 0).float()[:, None]
    if weights is not None:
        rows = rows * weights.reshape(-1, 1).float()
    return rows.view(tokens, top_k, -1).sum(1).to(src.dtype)


def scatter_rows(src, index, n_out):
    """out[index[i]] = src[i] for index[i] >= 0; rows of `out` that no index names are undefined
    on CUDA (callers name every row) and zero on the host."""
    if src.is_cuda:
        src = src.contiguous()
        out = torch.empty((n_out, src.shape[1]), dtype=src.dtype, device=src.device)
        with _lib.on_device(src.device):
            rc = _lib.load().stk_b200_scatter_rows(
                _lib.ptr(src), _lib.ptr(out), _lib.ptr(index), index.numel(),
                src.shape[1] * src.element_size(), _lib.stream_ptr(src.device))
        _lib.check(rc, "stk_b200_scatter_rows")
        return out
    out = src.new_zeros((n_out, src.shape[1]))
    valid = index >= 0
    out[index[valid].long()] = src[valid]
    return out


def bin_index(counts, total_padded, block=BLOCK, compose=None, inverse_size=None):
    """Gather index of the padded expert bins.

    counts: int64 [world, local_experts], rows received from each peer for each local expert (the
    received rows are ordered by peer, then expert).  Returns (index int32 [total_padded],
    bin_rows int32 [local_experts]); see stk_b200_bin_index in include/stk_b200.h.  With
    inverse_size = n a third result, position int32 [n], says where source row s went
    (index[position[s]] == s)."""
    world, local = counts.shape
    if counts.is_cuda:
        dev = counts.device
        index = torch.empty(total_padded, dtype=torch.int32, device=dev)
        bin_rows = torch.empty(local, dtype=torch.int32, device=dev)
        inverse = None if inverse_size is None else torch.full((inverse_size,), -1, dtype=torch.int32, device=dev)
        counts = counts.contiguous()
        with _lib.on_device(dev):
            rc = _lib.load().stk_b200_bin_index(
                _lib.ptr(counts), world, local, block, _lib.ptr(compose),
                _lib.ptr(index), total_padded, _lib.ptr(bin_rows), _lib.ptr(inverse), _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_bin_index")
        return (index, bin_rows) if inverse_size is None else (index, bin_rows, inverse)
    per_expert = counts.sum(0)
    padded = ((per_expert + block - 1) // block) * block
    index = torch.full((total_padded,), -1, dtype=torch.int32)
    seg = counts.reshape(-1)
    src_start = (torch.cumsum(seg, 0) - seg).view(world, local)
    bin_start = torch.cumsum(padded, 0) - padded
    for e in range(local):
        pos = int(bin_start[e])
        for p in range(world):
            n = int(counts[p, e])
            index[pos:pos + n] = torch.arange(int(src_start[p, e]), int(src_start[p, e]) + n,
                                              dtype=torch.int32)
            pos += n
    if compose is not None:
        valid = index >= 0
        index[valid] = compose[index[valid].long()]
    bin_rows = (padded // block).to(torch.int32)
    if inverse_size is None:
        return index, bin_rows
    inverse = torch.full((inverse_size,), -1, dtype=torch.int32)
    valid = index >= 0
    inverse[index[valid].long()] = torch.nonzero(valid).view(-1).to(torch.int32)
    return index, bin_rows, inverse


def padded_bins(counts, block=BLOCK):
    """(padded counts, exclusive start of every expert's padded bin, total padded rows)."""
    padded = ((counts + block - 1) // block) * block
    starts = torch.cumsum(padded, 0) - padded
    return padded, starts, int(padded.sum().item())


def topology_from_bins(bin_rows, block_rows, ffn, dtype, device, block=BLOCK, data=None, materialize=True):
    """stk.Matrix [block_rows*128, E*ffn]: expert e owns bin_rows[e] consecutive block rows and its
    own ffn/128 block columns.  bin_rows: int32 [E] on `device`; block_rows: their sum, known to the
    host.  All seven metadata arrays are written by one kernel (the transposed ones in closed
    form, nothing is sorted).  materialize=False: the values are a stride-0 placeholder of the right
    shape that occupies no memory - enough for stk.ops.sdd, which only takes the shape from it."""
    experts = bin_rows.numel()
    cpb = ffn // block
    nnz = block_rows * cpb
    meta16 = torch.empty((3, max(nnz, 1)), dtype=_kernels.index_dtype_for(block_rows, experts * cpb), device=device)
    offsets = torch.empty(block_rows + 1, dtype=torch.int32, device=device)
    offsets_t = torch.empty(experts * cpb + 1, dtype=torch.int32, device=device)
    block_offsets_t = torch.empty(nnz, dtype=torch.int32, device=device)
    row_idx, col_idx, col_idx_t = (meta16[i, :nnz] for i in range(3))
    with _lib.on_device(device):
        rc = _lib.entry("stk_b200_dmoe_topology", meta16)(
            _lib.ptr(bin_rows), experts, cpb, block_rows, _lib.ptr(row_idx), _lib.ptr(col_idx),
            _lib.ptr(offsets), _lib.ptr(col_idx_t), _lib.ptr(offsets_t), _lib.ptr(block_offsets_t),
            _lib.stream_ptr(device))
    _lib.check(rc, "stk_b200_dmoe_topology")
    if data is None:
        data = (torch.empty((nnz, block, block), dtype=dtype, device=device) if materialize
                else torch.empty((), dtype=dtype, device=device).expand(nnz, block, block))
    if cpb % 2 == 0:
        # Known by construction: all block rows of an expert share one column list and column
        # pairs never straddle experts; only row pairs at expert boundaries fail to pair.
        _kernels.set_pair_hints(col_idx, 0.9, 1.0, 0.9, True)
    return Matrix(torch.Size((block_rows * block, experts * ffn)), data, row_idx, col_idx, offsets,
                  col_idx_t, offsets_t, block_offsets_t)


def block_diagonal_topology(padded_counts, ffn, dtype, device, block=BLOCK, data=None):
    """Same topology from per-expert padded row counts (host or device tensor)."""
    bin_rows = (padded_counts // block).to(torch.int32)
    block_rows = int(bin_rows.sum())
    return topology_from_bins(bin_rows.to(device), block_rows, ffn, dtype, device, block, data)


_READ_BACK_BUFFERS = {}


def read_back(t):
    """Host copy of a small device tensor (waits for the current stream).  A kernel writes it into
    pinned host memory, so the read-back does not queue behind large copies on the copy engine;
    host tensors are returned as they are.  The returned tensor is a fresh one."""
    if not t.is_cuda:
        return t
    t = t.contiguous()
    nbytes = t.numel() * t.element_size()
    key = (t.device, max(256, 1 << (nbytes - 1).bit_length()) if nbytes else 256)
    buf = _READ_BACK_BUFFERS.get(key)
    if buf is None:
        buf = _READ_BACK_BUFFERS[key] = torch.empty(key[1], dtype=torch.uint8).pin_memory()
    with _lib.on_device(t.device):
        rc = _lib.load().stk_b200_copy_bytes(_lib.ptr(t), buf.data_ptr(), nbytes, _lib.stream_ptr(t.device))
    _lib.check(rc, "stk_b200_copy_bytes")
    torch.cuda.current_stream(t.device).synchronize()
    return buf[:nbytes].clone().view(t.dtype).view(t.shape)


# ------------------------------------------------------------------------------ one GPU
def _flat_slots(expert_ids):
    """(flat expert id per slot, k): expert_ids is [T] (top-1) or [T, k]; slot = token * k + choice."""
    if expert_ids.dim() == 1:
        return expert_ids, 1
    return expert_ids.reshape(-1), expert_ids.shape[1]


def route_topk(expert_ids, num_experts, block=BLOCK):
    """Placement of the (token, choice) slots of top-k routing in padded expert order on one device.

    expert_ids: [T] or [T, k].  Returns (index, position, padded, bin_rows, total): padded row r
    holds slot index[r] (zero padding where index[r] < 0); slot s sits in padded row position[s];
    padded = rows per expert bin (host int64 [E]); bin_rows = the same in blocks, on the device."""
    flat, _ = _flat_slots(expert_ids)
    order, offsets = sort_by_expert(flat, num_experts)
    counts = (offsets[1:] - offsets[:-1]).to(torch.int64).view(1, num_experts)
    host_counts = read_back(counts).view(-1)               # the one synchronisation
    padded = ((host_counts + block - 1) // block) * block
    total = int(padded.sum())
    index, bin_rows, position = bin_index(counts, total, block, compose=order, inverse_size=flat.numel())
    return index, position, padded, bin_rows, total


def route_top1(expert_ids, num_experts, block=BLOCK):
    """route_topk for one choice per token, without the inverse: (index, padded, bin_rows, total)."""
    index, _, padded, bin_rows, total = route_topk(expert_ids, num_experts, block)
    return index, padded, bin_rows, total


def permute_tokens(x, index, total_rows=None, top_k=1):
    """Padded, expert-ordered copy of the token matrix x [T, h] (padding rows are zero); with top_k > 1
    `index` holds slots and every token's row is copied to each of its k places."""
    return gather_rows(x, index, total_rows, index_div=top_k)


def unpermute_tokens(y, index, tokens):
    """Inverse of permute_tokens for top-1 routing: token t gets the padded row that held it."""
    return scatter_rows(y, index, tokens)


def combine_tokens(y, position, weights, tokens, top_k):
    """Inverse of permute_tokens for top-k routing: out[t] = sum_j weights[t, j] * y[position[t*k + j]]."""
    return weighted_sum_rows(y, position, weights, tokens, top_k)


# ------------------------------------------------------------------------------ expert parallel
class ExpertParallelExchange:
    """Token exchange of an expert-parallel dMoE layer: rank g owns experts
    [g*E/n, (g+1)*E/n); every rank starts with its own tokens and their expert ids ([T] or, for
    top-k routing, [T, k]).

    dispatch(): the (token, choice) slots are sorted by expert (hence by destination rank), the
    per-expert counts are exchanged, and the rows travel with all_to_all_single; the receiver gathers
    them into per-expert bins padded to a multiple of 128 rows.  combine(): the inverse, with the k
    rows of a token summed under their weights.  One host read-back per dispatch (the counts: NCCL
    needs the split sizes on the host).  Works with any torch.distributed backend: NCCL over NVLink
    on the GPUs, gloo on the host for tests.
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
        """Returns (x_padded [T'_local, h], bin_rows int32 [local_experts] on x's device, state);
        state["block_rows"] is the number of padded block rows (host int)."""
        dev = x.device
        world, local = self.world, self.local_experts
        flat, top_k = _flat_slots(expert_ids)
        order, offsets = sort_by_expert(flat, self.num_experts)
        counts = torch.empty((2, self.num_experts), dtype=torch.int64, device=dev)
        counts[0] = offsets[1:] - offsets[:-1]
        # counts[0][e] for the experts of rank g go to rank g: one row of E/n counts per peer
        dist.all_to_all_single(counts[1], counts[0], group=self.group)
        host = read_back(counts)                              # the one synchronisation
        send_splits = host[0].view(world, local).sum(1).tolist()
        recv_by_peer = host[1].view(world, local)
        recv_splits = recv_by_peer.sum(1).tolist()
        per_expert = recv_by_peer.sum(0)
        total = int((((per_expert + self.block - 1) // self.block) * self.block).sum())
        recv = torch.empty((sum(recv_splits), x.shape[1]), dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv, gather_rows(x, order, index_div=top_k), recv_splits, send_splits,
                               group=self.group)
        index, bin_rows = bin_index(counts[1].view(world, local), total, self.block)
        x_padded = gather_rows(recv, index, total)
        state = dict(order=order, send_splits=send_splits, recv_splits=recv_splits, index=index,
                     received=recv.shape[0], tokens=x.shape[0], top_k=top_k, block_rows=total // self.block)
        return x_padded, bin_rows, state

    def combine(self, y_padded, state, weights=None):
        """Inverse of dispatch for the per-slot results y_padded [T'_local, h_out]: token t gets
        sum_j weights[t, j] * (result of its j-th slot); weights None = ones."""
        slots = state["tokens"] * state["top_k"]
        back = scatter_rows(y_padded, state["index"], state["received"])
        out_sorted = torch.empty((slots, y_padded.shape[1]), dtype=y_padded.dtype, device=y_padded.device)
        dist.all_to_all_single(out_sorted, back, state["send_splits"], state["recv_splits"],
                               group=self.group)
        by_slot = scatter_rows(out_sorted, state["order"], slots)
        if state["top_k"] == 1 and weights is None:
            return by_slot
        return weighted_sum_rows(by_slot, None, weights, state["tokens"], state["top_k"])


# ------------------------------------------------------------------------------ exchange over peer memory
def _ep_call(name, device, *args):
    with _lib.on_device(device):
        rc = getattr(_lib.load(), name)(*args, _lib.stream_ptr(device))
    _lib.check(rc, name)


class PeerExchangeBuffers:
    """One rank's share of the exchange state.  Written by the peers: the count matrix, the padded
    bins (token rows and their tags), the slot-ordered rows that come back, and two flag arrays for
    the barriers.  `peer_*` are int64 device arrays with the address of the same region on every
    rank, as mapped in this process."""

    def __init__(self, counts, recv, tags, slots, peer_counts, peer_recv, peer_tags, peer_slots,
                 peer_flags=(None, None)):
        self.counts, self.recv, self.tags, self.slots = counts, recv, tags, slots
        self.peer_counts, self.peer_recv, self.peer_tags, self.peer_slots = peer_counts, peer_recv, peer_tags, peer_slots
        self.peer_flags = peer_flags


class PeerExchange:
    """ExpertParallelExchange with this library's own kernels moving the rows over NVLink.

    Every rank pushes the token row of each of its (token, choice) slots straight into the padded bin
    of the slot's expert on the rank that owns it, tagged with where it came from; after the
    experts' MLP the owner pushes every result row back into the home rank's slot-ordered buffer,
    where the k rows of a token are summed under their weights.  Only stores cross NVLink.  The
    buffers live in torch symmetric memory, allocated once for `capacity_rows` padded rows; there is
    no NCCL call in a step: the per-expert counts travel the same way, and the phases are separated by
    the library's own barrier kernel (bounded wait).  One host read-back per dispatch (the padded row
    counts, which size the topology).  Same results as ExpertParallelExchange.

    chunks > 1 cuts every rank's local experts into that many groups; forward() then overlaps the
    exchange of one group with the products of another on a second stream.

    `buffers` / `barrier` can be given to run several ranks of this logic inside one process on one
    GPU (tests): then nothing is allocated here and `barrier(channel)` is called where ranks meet.
    """

    BARRIER_TIMEOUT_MS = 20000

    def __init__(self, num_experts, tokens, hidden, out_hidden, dtype, device, group=None,
                 block=BLOCK, capacity_rows=None, world=None, rank=None, buffers=None, barrier=None,
                 top_k=1, chunks=1):
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts, self.local_experts = num_experts, num_experts // self.world
        if not 1 <= chunks <= min(self.local_experts, 8):
            raise ValueError(f"chunks must lie in 1..min(local experts, 8), got {chunks}")
        self.block, self.device, self.dtype = block, torch.device(device), dtype
        self.hidden, self.out_hidden, self.top_k, self.chunks = hidden, out_hidden, top_k, chunks
        self.slot_rows = tokens * top_k
        if capacity_rows is None:
            capacity_rows = 2 * self.slot_rows + self.local_experts * block
        self.capacity_rows = (capacity_rows + block - 1) // block * block
        if buffers is None:
            # symmetric allocations have the same size on every rank
            cap = torch.tensor([self.capacity_rows, self.slot_rows], dtype=torch.int64, device=self.device)
            dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=group)
            self.capacity_rows, self.slot_rows = int(cap[0]), int(cap[1])
            buffers = self._allocate(group)
        if barrier is None:
            barrier = self._barrier
        self.buf, self.barrier = buffers, barrier
        self.result = torch.empty((self.capacity_rows, out_hidden), dtype=dtype, device=self.device)
        self._totals_host = torch.zeros(3 + chunks, dtype=torch.int64).pin_memory()
        self._epoch = [0, 0]
        self._side = self._prep = None

    def _allocate(self, group):
        import torch.distributed._symmetric_memory as symm_mem
        elem = torch.empty((), dtype=self.dtype).element_size()
        align = lambda n: (n + 255) // 256 * 256
        sizes = [2 * 8 * 64,                                           # two flag arrays of 64 int64
                 4 * self.world * self.num_experts,                    # counts
                 self.capacity_rows * self.hidden * elem,              # recv
                 8 * self.capacity_rows,                               # tags
                 self.slot_rows * self.out_hidden * elem]              # slots
        offs = [0]
        for n in sizes:
            offs.append(offs[-1] + align(n))
        raw = symm_mem.empty(offs[-1], dtype=torch.uint8, device=self.device)
        raw[:offs[1]].zero_()
        torch.cuda.synchronize(self.device)
        handle = symm_mem.rendezvous(raw, group if group is not None else dist.group.WORLD)
        dist.barrier(group=group)                                     # everyone's flags are zero before anyone signals
        ptrs = [int(p) for p in handle.buffer_ptrs]
        dev_ptrs = lambda off: torch.tensor([p + off for p in ptrs], dtype=torch.int64, device=self.device)
        view = lambda i: raw[offs[i]:offs[i] + sizes[i]]
        counts = view(1).view(torch.int32).view(self.world, self.num_experts)
        recv = view(2).view(self.dtype).view(self.capacity_rows, self.hidden)
        tags = view(3).view(torch.int64)
        slots = view(4).view(self.dtype).view(self.slot_rows, self.out_hidden)
        self._raw, self._handle = raw, handle
        return PeerExchangeBuffers(counts, recv, tags, slots, dev_ptrs(offs[1]), dev_ptrs(offs[2]),
                                   dev_ptrs(offs[3]), dev_ptrs(offs[4]), (dev_ptrs(0), dev_ptrs(8 * 64)))

    def _barrier(self, channel):
        """All ranks meet on the current stream (channel 0: main stream, 1: the exchange stream)."""
        self._epoch[channel] += 1
        _ep_call("stk_b200_ep_barrier", self.device, _lib.ptr(self.buf.peer_flags[channel]), self.world,
                 self.rank, self._epoch[channel], self.BARRIER_TIMEOUT_MS)

    # The phases are separate methods so that a single-process emulation can interleave the ranks;
    # dispatch() / combine() / forward() run them in order with the barriers in between.
    def share_counts(self, expert_ids):
        flat, top_k = _flat_slots(expert_ids)
        if top_k != self.top_k:
            raise ValueError(f"exchange built for top-{self.top_k} routing, got {top_k} choices per token")
        order, offsets = sort_by_expert(flat, self.num_experts)
        _ep_call("stk_b200_ep_share_counts", self.device, _lib.ptr(offsets), _lib.ptr(self.buf.peer_counts),
                 self.world, self.num_experts, self.rank)
        return order, offsets

    def plan(self):
        """After the counts of all ranks have arrived: where this rank's rows go, this rank's bins,
        the padded row counts (copied to pinned host memory by a kernel), zeroed padding rows."""
        dev = self.device
        dest_base = torch.empty(self.num_experts, dtype=torch.int64, device=dev)
        bin_rows = torch.empty(self.local_experts, dtype=torch.int32, device=dev)
        totals = torch.empty(3 + self.chunks, dtype=torch.int64, device=dev)
        _ep_call("stk_b200_ep_plan", dev, _lib.ptr(self.buf.counts), self.world, self.num_experts, self.rank,
                 self.block, self.chunks, _lib.ptr(dest_base), _lib.ptr(bin_rows), _lib.ptr(totals))
        with _lib.on_device(dev):        # by a kernel, not the copy engine (see read_back)
            rc = _lib.load().stk_b200_copy_bytes(_lib.ptr(totals), self._totals_host.data_ptr(),
                                                 8 * (3 + self.chunks), _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_copy_bytes")
        elem = self.buf.recv.element_size()
        _ep_call("stk_b200_ep_zero_padding", dev, _lib.ptr(self.buf.counts), self.world, self.num_experts,
                 self.rank, self.block, _lib.ptr(self.buf.recv), _lib.ptr(self.buf.tags), self.hidden * elem,
                 self.capacity_rows)
        self._planned = torch.cuda.Event()
        self._planned.record(torch.cuda.current_stream(dev))
        return dest_base, bin_rows

    def push(self, x, order, offsets, dest_base, chunk=0, chunks=1):
        """This rank's rows (of the experts in `chunk` of every owner) into the owners' bins."""
        x = x.contiguous()
        _ep_call("stk_b200_ep_dispatch", self.device, _lib.ptr(x), _lib.ptr(order), _lib.ptr(offsets),
                 _lib.ptr(dest_base), _lib.ptr(self.buf.peer_recv), _lib.ptr(self.buf.peer_tags),
                 order.numel(), self.top_k, self.world, self.num_experts, self.rank, chunk, chunks,
                 self.hidden * x.element_size(), self.capacity_rows)
        return x

    def totals(self):
        """Host values (padded rows of this rank, rows received, largest padded row count of any
        rank, padded rows per chunk); waits for plan() only.  Every rank sees the same largest count,
        so if the buffers of ANY rank are too small every rank raises here, before the next barrier."""
        self._planned.synchronize()                                    # the one synchronisation
        t = [int(v) for v in self._totals_host]
        if t[2] > self.capacity_rows:
            raise RuntimeError(f"{t[2]} padded rows arrive at one rank but the exchange buffers hold "
                               f"{self.capacity_rows}: construct PeerExchange with a larger capacity_rows")
        return t

    def padded_rows(self):
        return self.totals()[0]

    def dispatch(self, x, expert_ids):
        """Returns (x_padded [T'_local, h] - a view of the receive buffer, valid until the next
        dispatch -, bin_rows int32 [local_experts], state)."""
        order, offsets = self.share_counts(expert_ids)
        self.barrier(0)
        dest_base, bin_rows = self.plan()
        keep = self.push(x, order, offsets, dest_base)
        self.barrier(0)                  # enqueued before the read-back: it runs while the host wakes up
        t = self.totals()
        state = dict(tokens=x.shape[0], block_rows=t[0] // self.block, total=t[0], keep=keep)
        return self.buf.recv[:t[0]], bin_rows, state

    def result_rows(self, state):
        """Where the experts' output rows of this dispatch belong: write them here (e.g.
        stk.ops.dsd(h, w2, out=...)) and combine() has nothing to copy."""
        return self.result[:state["total"]]

    def give_back(self, row0, n_rows):
        """Result rows [row0, row0 + n_rows) travel to the slot-ordered buffers of their home ranks."""
        _ep_call("stk_b200_ep_return", self.device, _lib.ptr(self.result), _lib.ptr(self.buf.tags),
                 _lib.ptr(self.buf.peer_slots), row0, n_rows, self.world,
                 self.out_hidden * self.result.element_size(), self.slot_rows)

    def gather_slots(self, tokens, weights=None):
        """out[t] = sum_j weights[t, j] * (row that came back for slot t*k + j)."""
        return weighted_sum_rows(self.buf.slots, None, weights, tokens, self.top_k)

    def combine(self, y_padded, state, weights=None):
        """Inverse of dispatch for the per-slot results y_padded [T'_local, out_hidden]."""
        target = self.result_rows(state)
        if y_padded.data_ptr() != target.data_ptr():
            target.copy_(y_padded)
        self.give_back(0, state["total"])
        self.barrier(0)
        return self.gather_slots(state["tokens"], weights)

    def forward(self, x, expert_ids, weights, expert_fn, prepare_fn=None):
        """One expert-parallel step with the exchange overlapped chunk by chunk.

        expert_fn(chunk, x_rows, bin_rows, block_rows, out_rows) runs the experts' MLP of one chunk:
        x_rows [rows, hidden] are the padded bins of the chunk's experts (bin_rows int32 on the
        device, one entry per expert of the chunk; block_rows their sum, a host int) and the result
        goes into out_rows [rows, out_hidden].  While chunk c is computed on the current stream, the
        rows of chunk c + 1 arrive and the results of chunk c - 1 travel home on a second stream.

        prepare_fn(chunk, bin_rows, block_rows), optional, is called for every chunk as soon as the
        bin sizes are known, before any rows are waited for, and what it returns is handed to
        expert_fn as a sixth argument: the place for work that depends on the bin sizes only (the
        chunk's topology, the pair kernel's work-item table), which would otherwise sit between the
        products of one chunk and the next."""
        dev, chunks = self.device, self.chunks
        if self._side is None:
            self._side = torch.cuda.Stream(dev)
        main, side = torch.cuda.current_stream(dev), self._side
        order, offsets = self.share_counts(expert_ids)
        self.barrier(0)
        dest_base, bin_rows = self.plan()
        side.wait_event(self._planned)
        pushed = []
        with torch.cuda.stream(side):
            for c in range(chunks):
                keep = self.push(x, order, offsets, dest_base, c, chunks)
                self.barrier(1)
                ev = torch.cuda.Event()
                ev.record(side)
                pushed.append(ev)
        for used_on_side in (keep, order, offsets, dest_base):
            used_on_side.record_stream(side)
        t = self.totals()
        per = self.local_experts
        bounds = [(-(-c * per // chunks), -(-(c + 1) * per // chunks)) for c in range(chunks)]  # le*chunks//per == c
        prepared, ready = [None] * chunks, [None] * chunks

        def prepare(c):
            # chunk 0 on the current stream (its products come next); the others on a stream of their
            # own, issued right after the products of the chunk before them, so that they run beside
            # those products and the host never keeps the first products waiting
            if prepare_fn is None or not t[3 + c]:
                return
            e0, e1 = bounds[c]
            with torch.cuda.stream(main if c == 0 else self._prep):
                prepared[c] = prepare_fn(c, bin_rows[e0:e1], t[3 + c] // self.block)
                if c:
                    ready[c] = torch.cuda.Event()
                    ready[c].record(self._prep)

        if prepare_fn is not None:
            if self._prep is None:
                self._prep = torch.cuda.Stream(dev)
            self._prep.wait_stream(main)
            prepare(0)
        row0 = 0
        for c in range(chunks):
            rows = t[3 + c]
            e0, e1 = bounds[c]
            main.wait_event(pushed[c])
            if ready[c] is not None:
                main.wait_event(ready[c])
            if rows:
                extra = () if prepare_fn is None else (prepared[c],)
                expert_fn(c, self.buf.recv[row0:row0 + rows], bin_rows[e0:e1], rows // self.block,
                          self.result[row0:row0 + rows], *extra)
            if c + 1 < chunks:
                prepare(c + 1)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(side):
                side.wait_event(done)
                self.give_back(row0, rows)
            row0 += rows
        with torch.cuda.stream(side):
            self.barrier(1)
            home = torch.cuda.Event()
            home.record(side)
        main.wait_event(home)
        if prepare_fn is not None:
            # what prepare_fn allocated on its stream was read by the products on the current one: the
            # stream's next allocations (which may reuse that memory) come after them
            self._prep.wait_stream(main)
        return self.gather_slots(x.shape[0], weights)


# ------------------------------------------------------------------------------ batches from host memory
def bind_host_to_gpu_node(device):
    """Restricts the calling process to the CPU cores next to `device` (the cores NVML reports for the GPU's
    NUMA node, intersected with the cores the process may use), so that pinned host buffers allocated
    afterwards and the copy threads live on that node: with one process per GPU, host <-> device copies of
    several ranks then do not cross the socket interconnect.  Only reads NVML; changes this process's
    scheduling affinity, nothing of the GPU's.  Returns the number of cores kept, or 0 when nothing was changed
    (NVML or the affinity call unavailable, or the GPU's cores are not among the allowed ones)."""
    import os
    try:
        import pynvml
        device = torch.device(device)
        props = torch.cuda.get_device_properties(device)
        pynvml.nvmlInit()
        try:
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(
                f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0".encode())
            words = (os.cpu_count() + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        finally:
            pynvml.nvmlShutdown()
        near = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        keep = near & os.sched_getaffinity(0)
        if not keep or keep == os.sched_getaffinity(0):
            return 0
        os.sched_setaffinity(0, keep)
        return len(keep)
    except Exception:          # no NVML, no such call on this platform, not permitted: leave the process as it is
        return 0


class HostPipeline:
    """Feeds a device step with batches that live in pinned host memory and returns its results to
    pinned host memory, with the copies of neighbouring batches overlapping the step: the inputs of
    batch i+1 travel to the device (copy-in stream) and the result of batch i-1 travels back
    (copy-out stream) while batch i is computed on the current stream.  Two device input buffers
    and two host result buffers are reused in turn.

        pipe = HostPipeline(step, device)              # step(*device_inputs) -> device tensor
        for batch in batches:                          # batch: tuple of pinned host tensors
            done = pipe.submit(*batch)                 # result of the PREVIOUS batch, or None
        last = pipe.flush()

    submit() returns the host tensor holding the previous batch's result; it is valid once
    `pipe.wait(done)` has returned (or after flush()) and until two more batches were submitted.
    """

    def __init__(self, step, device):
        self.step, self.device = step, torch.device(device)
        self.copy_in, self.copy_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.inputs = [None, None]           # device input buffers
        self.results = [None, None]          # pinned host result buffers
        self.in_ready = [torch.cuda.Event() for _ in range(2)]
        self.in_free = [None, None]
        self.out_ready = [None, None]
        self.count = 0                       # batches submitted
        self.pending = None                  # slot whose inputs are on their way but not yet computed

    def _upload(self, slot, host_tensors):
        bufs = self.inputs[slot]
        stale = bufs is None or len(bufs) != len(host_tensors) or any(
            b.shape != t.shape or b.dtype != t.dtype for b, t in zip(bufs, host_tensors))
        if stale:
            # New buffers may reuse memory that kernels queued on the current stream still read: the
            # copy-in stream first catches up with it, and the buffers belong to the copy-in stream.
            self.copy_in.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.copy_in):
                self.inputs[slot] = [torch.empty(t.shape, dtype=t.dtype, device=self.device)
                                     for t in host_tensors]
        with torch.cuda.stream(self.copy_in):
            if self.in_free[slot] is not None:
                self.copy_in.wait_event(self.in_free[slot])     # the step that read this buffer is done
            for dst, src in zip(self.inputs[slot], host_tensors):
                dst.copy_(src, non_blocking=True)
            self.in_ready[slot].record(self.copy_in)

    def _compute(self, slot):
        main = torch.cuda.current_stream(self.device)
        main.wait_event(self.in_ready[slot])
        out = self.step(*self.inputs[slot])
        self.in_free[slot] = torch.cuda.Event()
        self.in_free[slot].record(main)
        done = torch.cuda.Event()
        done.record(main)
        if self.results[slot] is None or self.results[slot].shape != out.shape:
            self.results[slot] = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(done)
            self.results[slot].copy_(out, non_blocking=True)
            self.out_ready[slot] = torch.cuda.Event()
            self.out_ready[slot].record(self.copy_out)
        out.record_stream(self.copy_out)
        return self.results[slot]

    def submit(self, *host_tensors):
        slot = self.count % 2
        self._upload(slot, host_tensors)            # first, so that it overlaps the step below
        previous = self._compute(self.pending) if self.pending is not None else None
        self.pending = slot
        self.count += 1
        return previous

    def flush(self):
        """Computes the last submitted batch; returns its host result after all copies are done."""
        last = self._compute(self.pending) if self.pending is not None else None
        self.pending = None
        torch.cuda.current_stream(self.device).wait_stream(self.copy_out)
        self.copy_out.synchronize()
        return last

    def wait(self, host_result):
        for slot in range(2):
            if self.results[slot] is host_result and self.out_ready[slot] is not None:
                self.out_ready[slot].synchronize()


# ------------------------------------------------------------------------------ the experts' MLP, fused
class _ExpertMLP(torch.autograd.Function):
    """y = dsd(GeLU(sdd(x, w1, topo)), w2) with both element-wise steps inside the products'
    epilogues: the forward SDD writes the pre-activations and their GeLU in one pass, and the
    backward SDD (dy @ w2^T on the topology) multiplies by GeLU'(pre-activations) before it stores,
    so the hidden-size tensors are never read or written by an element-wise kernel."""

    @staticmethod
    def forward(ctx, x, w1, w2, shape, offsets, row_indices, column_indices, offsets_t,
                column_indices_t, block_offsets_t):
        meta = (offsets, row_indices, column_indices, offsets_t, column_indices_t, block_offsets_t)
        nnz = row_indices.numel()
        pre = torch.empty((nnz, BLOCK, BLOCK), dtype=x.dtype, device=x.device)
        act = torch.empty_like(pre)
        _kernels.sdd(x, w1, shape, pre, offsets, row_indices, column_indices, epilogue=2, aux=act)
        y = torch.empty((shape[0], w2.shape[1]), dtype=x.dtype, device=x.device)
        _kernels.dsd(shape, act, *meta, False, w2, y)
        ctx.save_for_backward(x, w1, w2, pre, act, *meta)
        ctx.shape = tuple(shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, pre, act = ctx.saved_tensors[:5]
        meta = ctx.saved_tensors[5:]
        offsets, row_indices, column_indices = meta[:3]
        shape = ctx.shape
        dy = dy.contiguous()
        dx = dw1 = dw2 = None
        if ctx.needs_input_grad[2]:
            dw2 = torch.empty_like(w2)                      # act^T @ dy
            _kernels.dsd((shape[1], shape[0]), act, *meta, True, dy, dw2)
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            d_pre = torch.empty_like(pre)                   # (dy @ w2^T) * GeLU'(pre), one kernel
            _kernels.sdd(dy, w2.t(), shape, d_pre, offsets, row_indices, column_indices, epilogue=3, aux=pre)
            if ctx.needs_input_grad[0]:
                dx = torch.empty_like(x)                    # d_pre @ w1^T
                _kernels.dsd(shape, d_pre, *meta, False, w1.t(), dx)
            if ctx.needs_input_grad[1]:
                dw1 = torch.empty_like(w1)                  # x^T @ d_pre
                _kernels.dds(x.t(), shape, d_pre, *meta, False, dw1)
        return (dx, dw1, dw2) + (None,) * 7


def expert_mlp(x, w1, w2, topo):
    """The experts' two-layer MLP of a dMoE layer on tokens in padded expert order:
    y = dsd(GeLU(sdd(x, w1, topo)), w2), differentiable in x, w1 and w2, with GeLU and its
    backward fused into the block-sparse products (see _ExpertMLP).  x [T', h], w1 [h, E*f],
    w2 [E*f, h_out] on the GPU, fp16 or bf16; topo: the block-diagonal topology of the batch."""
    assert isinstance(topo, Matrix) and topo.is_contiguous()
    return _ExpertMLP.apply(x.contiguous(), w1, w2, tuple(topo.size()), topo.offsets, topo.row_indices,
                            topo.column_indices, topo.offsets_t, topo.column_indices_t, topo.block_offsets_t)
