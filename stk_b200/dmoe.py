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
    """Stable sort of token indices by expert: (order int32 [T], offsets int32 [E+1])."""
    if expert_ids.is_cuda:
        ids16 = expert_ids.to(torch.int16)
        _, offsets, order = _kernels.transpose_meta(ids16, ids16, num_experts)
        return order, offsets
    order = torch.argsort(expert_ids, stable=True).to(torch.int32)
    counts = torch.bincount(expert_ids, minlength=num_experts)
    offsets = torch.cat([counts.new_zeros(1), torch.cumsum(counts, 0)]).to(torch.int32)
    return order, offsets


def gather_rows(src, index, n_out=None):
    """out[i] = src[index[i]], or a zero row where index[i] < 0."""
    n_out = index.numel() if n_out is None else n_out
    if src.is_cuda:
        src = src.contiguous()
        out = torch.empty((n_out, src.shape[1]), dtype=src.dtype, device=src.device)
        with _lib.on_device(src.device):
            rc = _lib.load().stk_b200_gather_rows(
                _lib.ptr(src), _lib.ptr(out), _lib.ptr(index), n_out,
                src.shape[1] * src.element_size(), _lib.stream_ptr(src.device))
        _lib.check(rc, "stk_b200_gather_rows")
        return out
    out = src.new_zeros((n_out, src.shape[1]))
    valid = index >= 0
    out[valid] = src[index[valid].long()]
    return out


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


def bin_index(counts, total_padded, block=BLOCK, compose=None):
    """Gather index of the padded expert bins.

    counts: int64 [world, local_experts], rows received from each peer for each local expert (the
    received rows are ordered by peer, then expert).  Returns (index int32 [total_padded],
    bin_rows int32 [local_experts]); see stk_b200_bin_index in include/stk_b200.h."""
    world, local = counts.shape
    if counts.is_cuda:
        dev = counts.device
        index = torch.empty(total_padded, dtype=torch.int32, device=dev)
        bin_rows = torch.empty(local, dtype=torch.int32, device=dev)
        with _lib.on_device(dev):
            rc = _lib.load().stk_b200_bin_index(
                _lib.ptr(counts.contiguous()), world, local, block, _lib.ptr(compose),
                _lib.ptr(index), total_padded, _lib.ptr(bin_rows), _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_bin_index")
        return index, bin_rows
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
    return index, (padded // block).to(torch.int32)


def padded_bins(counts, block=BLOCK):
    """(padded counts, exclusive start of every expert's padded bin, total padded rows)."""
    padded = ((counts + block - 1) // block) * block
    starts = torch.cumsum(padded, 0) - padded
    return padded, starts, int(padded.sum().item())


def topology_from_bins(bin_rows, block_rows, ffn, dtype, device, block=BLOCK, data=None):
    """stk.Matrix [block_rows*128, E*ffn]: expert e owns bin_rows[e] consecutive block rows and its
    own ffn/128 block columns.  bin_rows: int32 [E] on `device`; block_rows: their sum, known to the
    host.  All seven metadata arrays are written by one kernel (the transposed ones in closed
    form, nothing is sorted)."""
    experts = bin_rows.numel()
    cpb = ffn // block
    nnz = block_rows * cpb
    meta16 = torch.empty((3, max(nnz, 1)), dtype=torch.int16, device=device)
    offsets = torch.empty(block_rows + 1, dtype=torch.int32, device=device)
    offsets_t = torch.empty(experts * cpb + 1, dtype=torch.int32, device=device)
    block_offsets_t = torch.empty(nnz, dtype=torch.int32, device=device)
    row_idx, col_idx, col_idx_t = (meta16[i, :nnz] for i in range(3))
    with _lib.on_device(device):
        rc = _lib.load().stk_b200_dmoe_topology(
            _lib.ptr(bin_rows), experts, cpb, block_rows, _lib.ptr(row_idx), _lib.ptr(col_idx),
            _lib.ptr(offsets), _lib.ptr(col_idx_t), _lib.ptr(offsets_t), _lib.ptr(block_offsets_t),
            _lib.stream_ptr(device))
    _lib.check(rc, "stk_b200_dmoe_topology")
    if data is None:
        data = torch.empty((nnz, block, block), dtype=dtype, device=device)
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
def route_top1(expert_ids, num_experts, block=BLOCK):
    """Placement of tokens in padded expert order for top-1 routing on one device.

    Returns (index, padded, bin_rows, total): padded row r holds token index[r] (or is zero
    padding where index[r] < 0); padded = rows per expert bin (host int64 [E]); bin_rows = the same
    in blocks, on the device."""
    order, offsets = sort_by_expert(expert_ids, num_experts)
    counts = (offsets[1:] - offsets[:-1]).to(torch.int64).view(1, num_experts)
    host_counts = read_back(counts).view(-1)               # the one synchronisation
    padded = ((host_counts + block - 1) // block) * block
    total = int(padded.sum())
    index, bin_rows = bin_index(counts, total, block, compose=order)
    return index, padded, bin_rows, total


def permute_tokens(x, index, total_rows=None):
    """Padded, expert-ordered copy of the token matrix x [T, h] (padding rows are zero)."""
    return gather_rows(x, index, total_rows)


def unpermute_tokens(y, index, tokens):
    """Inverse of permute_tokens: token t gets the padded row that held it."""
    return scatter_rows(y, index, tokens)


# ------------------------------------------------------------------------------ expert parallel
class ExpertParallelExchange:
    """Token exchange of an expert-parallel dMoE layer: rank g owns experts
    [g*E/n, (g+1)*E/n); every rank starts with its own tokens and their expert ids.

    dispatch(): tokens are sorted by expert (hence by destination rank), the per-expert counts are
    exchanged, and the rows travel with all_to_all_single; the receiver gathers them into
    per-expert bins padded to a multiple of 128 rows.  combine(): the inverse.  One host read-back
    per dispatch (the counts: NCCL needs the split sizes on the host).  Works with any
    torch.distributed backend: NCCL over NVLink on the GPUs, gloo on the host for tests.
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
        order, offsets = sort_by_expert(expert_ids, self.num_experts)
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
        dist.all_to_all_single(recv, gather_rows(x, order), recv_splits, send_splits,
                               group=self.group)
        index, bin_rows = bin_index(counts[1].view(world, local), total, self.block)
        x_padded = gather_rows(recv, index, total)
        state = dict(order=order, send_splits=send_splits, recv_splits=recv_splits, index=index,
                     received=recv.shape[0], tokens=x.shape[0], block_rows=total // self.block)
        return x_padded, bin_rows, state

    def combine(self, y_padded, state):
        """Inverse of dispatch for the per-token results y_padded [T'_local, h_out]."""
        back = scatter_rows(y_padded, state["index"], state["received"])
        out_sorted = torch.empty((state["tokens"], y_padded.shape[1]), dtype=y_padded.dtype,
                                 device=y_padded.device)
        dist.all_to_all_single(out_sorted, back, state["send_splits"], state["recv_splits"],
                               group=self.group)
        return scatter_rows(out_sorted, state["order"], state["tokens"])


# ------------------------------------------------------------------------------ exchange over peer memory
def _ep_call(name, device, *args):
    with _lib.on_device(device):
        rc = getattr(_lib.load(), name)(*args, _lib.stream_ptr(device))
    _lib.check(rc, name)


class PeerExchangeBuffers:
    """One rank's share of the exchange state: the count matrix, the padded bins the peers push token
    rows into, and the result rows the peers pull from.  `peer_*` are int64 device arrays with the
    address of the same region on every rank, as mapped in this process."""

    def __init__(self, counts, recv, result, peer_counts, peer_recv, peer_result):
        self.counts, self.recv, self.result = counts, recv, result
        self.peer_counts, self.peer_recv, self.peer_result = peer_counts, peer_recv, peer_result


class PeerExchange:
    """ExpertParallelExchange with this library's own kernels moving the rows over NVLink.

    Every rank pushes its token rows straight into the padded expert bins of the rank that owns
    the expert (peer stores) and pulls its results from that rank's result buffer (peer loads); the
    buffers live in torch symmetric memory, allocated once for `capacity_rows` padded rows.  There
    is no NCCL call in a step: the per-expert counts travel the same way, and the steps are
    separated by the symmetric-memory barrier.  One host read-back per dispatch (the number of
    padded rows, which sizes the topology).  Same results, row for row, as ExpertParallelExchange.

    `buffers` / `barrier` can be given to run several ranks of this logic inside one process on one
    GPU (tests): then nothing is allocated here and `barrier()` is called where ranks must meet.
    """

    def __init__(self, num_experts, tokens, hidden, out_hidden, dtype, device, group=None,
                 block=BLOCK, capacity_rows=None, world=None, rank=None, buffers=None, barrier=None):
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts, self.local_experts = num_experts, num_experts // self.world
        self.block, self.device, self.dtype = block, torch.device(device), dtype
        self.hidden, self.out_hidden = hidden, out_hidden
        if capacity_rows is None:
            capacity_rows = 2 * tokens + self.local_experts * block
        self.capacity_rows = (capacity_rows + block - 1) // block * block
        if buffers is None:
            # symmetric allocations have the same size on every rank
            cap = torch.tensor([self.capacity_rows], dtype=torch.int64, device=self.device)
            dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=group)
            self.capacity_rows = int(cap.item())
            buffers, barrier = self._allocate(group)
        self.buf, self.barrier = buffers, barrier
        self._totals_host = torch.empty(2, dtype=torch.int64).pin_memory()

    def _allocate(self, group):
        import torch.distributed._symmetric_memory as symm_mem
        elem = torch.empty((), dtype=self.dtype).element_size()
        align = lambda n: (n + 255) // 256 * 256
        n_counts = align(4 * self.world * self.num_experts)
        n_recv = align(self.capacity_rows * self.hidden * elem)
        n_result = align(self.capacity_rows * self.out_hidden * elem)
        raw = symm_mem.empty(n_counts + n_recv + n_result, dtype=torch.uint8, device=self.device)
        handle = symm_mem.rendezvous(raw, group if group is not None else dist.group.WORLD)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        dev_ptrs = lambda off: torch.tensor([p + off for p in ptrs], dtype=torch.int64, device=self.device)
        counts = raw[:4 * self.world * self.num_experts].view(torch.int32).view(self.world, self.num_experts)
        recv = raw[n_counts:n_counts + self.capacity_rows * self.hidden * elem].view(self.dtype)
        result = raw[n_counts + n_recv:n_counts + n_recv + self.capacity_rows * self.out_hidden * elem].view(self.dtype)
        buffers = PeerExchangeBuffers(counts, recv.view(self.capacity_rows, self.hidden),
                                      result.view(self.capacity_rows, self.out_hidden),
                                      dev_ptrs(0), dev_ptrs(n_counts), dev_ptrs(n_counts + n_recv))
        self._raw, self._handle = raw, handle
        return buffers, handle.barrier

    # The three phases of dispatch are separate so that a single-process emulation can interleave
    # the ranks; dispatch() runs them back to back with the barriers in between.
    def share_counts(self, expert_ids):
        order, offsets = sort_by_expert(expert_ids, self.num_experts)
        _ep_call("stk_b200_ep_share_counts", self.device, _lib.ptr(offsets), _lib.ptr(self.buf.peer_counts),
                 self.world, self.num_experts, self.rank)
        return order, offsets

    def push(self, x, order, offsets):
        dev, tokens = self.device, x.shape[0]
        x = x.contiguous()
        dest_base = torch.empty(self.num_experts, dtype=torch.int64, device=dev)
        bin_rows = torch.empty(self.local_experts, dtype=torch.int32, device=dev)
        totals = torch.empty(2, dtype=torch.int64, device=dev)
        _ep_call("stk_b200_ep_plan", dev, _lib.ptr(self.buf.counts), self.world, self.num_experts, self.rank,
                 self.block, _lib.ptr(dest_base), _lib.ptr(bin_rows), _lib.ptr(totals))
        with _lib.on_device(dev):        # by a kernel, not the copy engine (see read_back)
            rc = _lib.load().stk_b200_copy_bytes(_lib.ptr(totals), self._totals_host.data_ptr(), 16,
                                                 _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_copy_bytes")
        row_bytes = self.hidden * x.element_size()
        _ep_call("stk_b200_ep_zero_padding", dev, _lib.ptr(self.buf.counts), self.world, self.num_experts,
                 self.rank, self.block, _lib.ptr(self.buf.recv), row_bytes, self.capacity_rows)
        dest = torch.empty(tokens, dtype=torch.int64, device=dev)
        _ep_call("stk_b200_ep_dispatch", dev, _lib.ptr(x), _lib.ptr(order), _lib.ptr(offsets),
                 _lib.ptr(dest_base), _lib.ptr(self.buf.peer_recv), tokens, self.world, self.num_experts,
                 row_bytes, self.capacity_rows, _lib.ptr(dest))
        return dest, bin_rows

    def padded_rows(self):
        """Host value of this rank's padded row count (waits for the stream)."""
        torch.cuda.current_stream(self.device).synchronize()       # the one synchronisation
        total = int(self._totals_host[0])
        if total > self.capacity_rows:
            raise RuntimeError(f"{total} padded rows arrive at rank {self.rank} but the exchange buffers hold "
                               f"{self.capacity_rows}: construct PeerExchange with a larger capacity_rows")
        return total

    def dispatch(self, x, expert_ids):
        """Returns (x_padded [T'_local, h] - a view of the receive buffer, valid until the next
        dispatch -, bin_rows int32 [local_experts], state)."""
        order, offsets = self.share_counts(expert_ids)
        self.barrier(0)
        dest, bin_rows = self.push(x, order, offsets)
        self.barrier(1)                  # enqueued before the read-back: it runs while the host wakes up
        total = self.padded_rows()
        state = dict(dest=dest, tokens=x.shape[0], block_rows=total // self.block, total=total)
        return self.buf.recv[:total], bin_rows, state

    def result_rows(self, state):
        """The rows of the result buffer for this dispatch: write the expert outputs here (e.g.
        stk.ops.dsd(h, w2, out=...)) and combine() has nothing to copy."""
        return self.buf.result[:state["total"]]

    def publish(self, y_padded, state):
        target = self.result_rows(state)
        if y_padded.data_ptr() != target.data_ptr():
            target.copy_(y_padded)

    def pull(self, state):
        out = torch.empty((state["tokens"], self.out_hidden), dtype=self.dtype, device=self.device)
        _ep_call("stk_b200_ep_combine", self.device, _lib.ptr(self.buf.peer_result), _lib.ptr(state["dest"]),
                 _lib.ptr(out), state["tokens"], self.out_hidden * out.element_size(), self.capacity_rows)
        return out

    def combine(self, y_padded, state):
        """Inverse of dispatch for the per-token results y_padded [T'_local, out_hidden]."""
        self.publish(y_padded, state)
        self.barrier(2)
        return self.pull(state)


# ------------------------------------------------------------------------------ batches from host memory
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
