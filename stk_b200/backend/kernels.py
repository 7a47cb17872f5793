"""Host launchers of the sm_100a kernels.

The four matmul / index launchers keep the names, argument order and meaning of the reference's
kernel backend (stk/backend/triton_kernels.py: dsd :222-276, dds :278-330, sdd :332-379,
row_indices :389-393), so the autograd glue above them is unchanged.  Three more launchers replace
what the reference composes from torch ops: transpose_meta (stk/matrix.py:105-123), the to_sparse
phases and to_dense (stk/ops/matrix_ops.py:36-85).

Everything here marshals tensors into the C ABI of libstk_b200.so; there is no other code path.
"""
import os

import torch

from stk_b200.backend import lib as _lib

BLOCK = 128  # the matmul kernels are built for 128x128 blocks

# Which matmul kernel runs: "0" = one 128x128 tile per CTA, "1" = 256x256 supertiles on CTA pairs
# wherever the metadata allows it, "2" = the same with 256x512 items for DSD / DDS, "3" = 128x256 tiles on one CTA (two blocks of a block row for SDD,
# one block row / column x 256 dense columns / rows for DSD / DDS), "auto" = per topology, from how
# well neighbouring block rows / columns pair up (see pair_hints).
PAIR_MODE = os.environ.get("STK_B200_PAIR_MODE", "auto")
# DSD / DDS on CTA pairs come in two tile shapes: 256x256 (two accumulators alternate, so the epilogue
# of one tile hides under the next tile's MMAs) and, mode "2", 256x512 (both accumulators belong to one
# tile: a quarter less operand traffic per FLOP, but the epilogue is exposed), which pays once the
# lists are long.  "auto" takes the wide shape from this many blocks per list on average.  Measured on
# dMoE topologies (8 experts x 4096 rows, 4096 dense columns) in loops of a second or more, i.e. under
# the power cap, wide against 256x256: 0.96 at 16 blocks per list, 0.99 - 1.02 at 32, 1.04 at 64, 1.06
# at 112 (in bursts of a few launches, where nothing is power-limited: 0.91 at 8, 0.98 at 16, 0.98 - 1.02
# from 32 on).
WIDE_MIN_LIST_BLOCKS = int(os.environ.get("STK_B200_WIDE_MIN_LIST_BLOCKS", "48"))
# ... and only when that gain survives the longer tail of half as many, twice as long items: the items
# are dealt in rounds over the CTA pairs, a launch lasts ceil(items / pairs) rounds, and the wide shape is
# taken when its share of useful rounds times WIDE_GAIN beats the 256x256 shape's (BASELINE configs[2],
# Zipf-imbalanced, 2048 dense columns: 524 wide items are 7.1 rounds of 74, i.e. 8, and ran 7 % behind
# 1048 narrow ones in 15).
WIDE_GAIN = 1.05
_PAIRS_RESIDENT = {}


def _pairs_resident(device):
    n = _PAIRS_RESIDENT.get(device)
    if n is None:
        n = _PAIRS_RESIDENT[device] = max(1, torch.cuda.get_device_properties(device).multi_processor_count // 2)
    return n
# DSD / DDS products that do not take the pair kernel run the 128x256 row kernel in these modes when
# the dense operand has at least 256 columns (DSD) / rows (DDS); "3" never takes the pair kernel.
ROW_KERNEL_MODES = ("3", "auto")
# SDD with the row kernel (two blocks of a block row per tile) has half as many, twice as long work
# items: on 8192^3 it is ahead of the 128x128 kernel from about 1000 blocks (level at 1024, 1190 vs
# 920 TFLOP/s at 2048) and behind at 512 (685 vs 750), where 256 items leave the 148 SMs unevenly loaded.
SDD_ROW_MIN_BLOCKS = 1536
# Fraction of the pair kernel's MMA work that must be useful for it to be chosen (measured with
# python -m stk_b200.benchmarks).  DSD / DDS ("rows", "cols"): the alternative is the 128x256 row
# kernel, which needs no pairing and is within 5 % of the pair kernel even on dMoE topologies
# (1300 vs 1390 TFLOP/s) and ahead of it as soon as a third of the pair kernel's work is wasted
# (1080 vs 920 at a useful share of 0.65), so only near-perfect pairings take the pair kernel.
# SDD ("tiles"): the alternative is the 128x128 kernel, still ahead at 0.53 (900 vs 690); dMoE
# topologies are above 0.9.
PAIR_THRESHOLD = {"rows": 0.85, "cols": 0.85, "tiles": 0.7}
_HINT_ATTR = "_stk_b200_pair_hints"
_PLAN_ATTR = "_stk_b200_pair_plan"


class _Hints:
    """What is known about how a topology pairs up; hangs on its column_indices tensor.

    values: (rows, cols, tiles, in_order, t_in_order) once known - useful fraction of the pair
    kernel's work when block rows / block columns / both are processed two at a time, whether the
    blocks are in ascending (row, column) order, and whether every block column's segment of
    column_indices_t ascends (None: not examined).  pending: a stats kernel that has been launched
    but whose result has not been read yet."""

    __slots__ = ("version", "values", "pending", "t_ptr")

    def __init__(self, version):
        self.version, self.values, self.pending, self.t_ptr = version, None, None, None


class _StatsSlots:
    """Pinned host memory the stats kernel writes its six numbers into: one arena, slots handed out in
    turn, so that asking about a topology allocates nothing and never waits for the device."""

    SLOTS, INTS = 1024, 8

    def __init__(self):
        self.arena = torch.zeros((self.SLOTS, self.INTS), dtype=torch.int32).pin_memory()
        self.next = 0

    def take(self):
        i = self.next % self.SLOTS
        self.next += 1
        self.arena[i].zero_()
        return self.next - 1, self.arena[i]

    def still_mine(self, ticket):
        return self.next - ticket <= self.SLOTS


_stats_slots = None


def set_pair_hints(column_indices, rows, cols, tiles, is_sorted=True, t_sorted=True):
    """Record how a topology pairs up, for callers that know it by construction.

    rows / cols / tiles: useful fraction of the pair kernel's work when block rows (2t, 2t+1),
    block columns (2u, 2u+1), or both, are processed together; is_sorted: blocks in ascending
    (row, column) order; t_sorted: every block column's rows ascend in column_indices_t."""
    h = _Hints(column_indices._version)
    h.values = (float(rows), float(cols), float(tiles), bool(is_sorted), bool(t_sorted))
    setattr(column_indices, _HINT_ATTR, h)


def _launch_stats(h, offsets, row_indices, column_indices, offsets_t, column_indices_t, block_cols):
    global _stats_slots
    if _stats_slots is None:
        _stats_slots = _StatsSlots()
    ticket, slot = _stats_slots.take()
    dev = column_indices.device
    row_indices, column_indices = row_indices.contiguous(), column_indices.contiguous()
    with _lib.on_device(dev):
        rc = _lib.entry("stk_b200_pair_stats", column_indices)(
            _lib.ptr(offsets), _lib.ptr(row_indices), _lib.ptr(column_indices), _lib.ptr(offsets_t),
            _lib.ptr(column_indices_t), offsets.numel() - 1, block_cols, column_indices.numel(),
            slot.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_pair_stats")
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(dev))
    h.pending = (ticket, slot, event, column_indices.numel())
    h.t_ptr = None if column_indices_t is None else column_indices_t.data_ptr()


def pair_hints(offsets, row_indices, column_indices, block_cols, offsets_t=None, column_indices_t=None,
               need_t=False, wait=False):
    """(rows, cols, tiles, in_order, t_in_order) of a topology, or None while that is not known yet.

    rows  = nnz / (2 * number of distinct (row pair, column) positions): DSD with S as stored,
            DDS with S transposed.
    cols  = nnz / (2 * distinct (row, column pair)): DSD with S transposed, DDS with S as stored.
    tiles = nnz / (4 * distinct (row pair, column pair)): SDD.
    Nothing here waits for the device (unless wait=True): the first question about an unknown
    topology launches one small kernel that writes its answer into pinned host memory, and the
    answer is picked up by whichever later call finds it complete; until then the caller gets None
    and runs a kernel that needs no pairing.  need_t: the caller pairs block COLUMNS and therefore
    needs the order inside column_indices_t examined as well."""
    h = getattr(column_indices, _HINT_ATTR, None)
    if h is None or h.version != column_indices._version:
        h = _Hints(column_indices._version)
        setattr(column_indices, _HINT_ATTR, h)
    if h.values is not None and not (need_t and h.values[4] is None):
        return h.values
    if column_indices.numel() == 0:
        h.values = (0.0, 0.0, 0.0, True, True)
        return h.values
    if h.pending is not None:
        ticket, slot, event, nnz = h.pending
        covers_t = h.t_ptr is not None and (column_indices_t is None or h.t_ptr == column_indices_t.data_ptr())
        if not _stats_slots.still_mine(ticket) or (need_t and not covers_t):
            h.pending = None
        else:
            if wait:
                event.synchronize()
            if not event.query():
                return None
            n_rp, n_cp, n_t, in_order, t_order = (int(v) for v in slot[:5])
            h.values = (nnz / (2.0 * max(n_rp, 1)), nnz / (2.0 * max(n_cp, 1)), nnz / (4.0 * max(n_t, 1)),
                        in_order == 1, None if t_order < 0 else t_order == 1)
            h.pending = None
            return h.values
    _launch_stats(h, offsets, row_indices, column_indices, offsets_t, column_indices_t, block_cols)
    if wait:
        return pair_hints(offsets, row_indices, column_indices, block_cols, offsets_t, column_indices_t,
                          need_t, wait)
    return None


def _use_pairs(kind, offsets, row_indices, column_indices, block_cols, offsets_t=None, column_indices_t=None):
    """kind: "rows", "cols" or "tiles" - which neighbours the product would pair.  1 = pair kernel."""
    if PAIR_MODE in ("0", "3"):
        return 0
    forced = PAIR_MODE in ("1", "2")
    hints = pair_hints(offsets, row_indices, column_indices, block_cols, offsets_t, column_indices_t,
                       need_t=kind == "cols", wait=forced)
    if hints is None:
        return 0
    rows, cols, tiles, in_order, t_order = hints
    # the merge walks need ascending columns inside every block row (and, when block columns are
    # paired, ascending rows inside every block column); anything else takes a kernel that does not
    if not in_order or (kind == "cols" and not t_order):
        return 0
    if forced:
        return 1
    return int({"rows": rows, "cols": cols, "tiles": tiles}[kind] >= PAIR_THRESHOLD[kind])


def _pair_shape(pairs, nnz, num_lists, dense_extent, device):
    """pair_mode of a DSD / DDS product that takes the pair kernel: 1 = 256x256 tiles, 2 = 256x512."""
    if pairs != 1:
        return pairs
    if PAIR_MODE == "2":
        return 2
    if PAIR_MODE == "auto" and nnz >= WIDE_MIN_LIST_BLOCKS * num_lists:
        pairs_on_gpu, groups = _pairs_resident(device), (num_lists + 1) // 2
        useful = lambda items: items / (pairs_on_gpu * -(-items // pairs_on_gpu))
        wide_items = groups * ((dense_extent + 4 * BLOCK - 1) // (4 * BLOCK))
        narrow_items = groups * ((dense_extent + 2 * BLOCK - 1) // (2 * BLOCK))
        if useful(wide_items) * WIDE_GAIN > useful(narrow_items):
            return 2
    return 1


def pair_plan(offsets, indices):
    """The pair kernel's work-item table for one family of lists - (offsets, column_indices) for
    block rows, (offsets_t, column_indices_t) for block columns -, computed once per topology by a
    small kernel on the current stream and kept on the index tensor."""
    cached = getattr(indices, _PLAN_ATTR, None)
    if cached is not None and cached[0] == (indices._version, offsets.data_ptr(), offsets._version):
        return cached[1]
    num_lists = offsets.numel() - 1
    lib = _lib.load()
    nbytes = lib.stk_b200_pair_plan_bytes(num_lists)
    plan = torch.empty(nbytes // 4, dtype=torch.int32, device=indices.device)
    with _lib.on_device(indices.device):
        rc = _lib.entry("stk_b200_pair_plan", indices)(_lib.ptr(offsets), _lib.ptr(indices), num_lists, _lib.ptr(plan), nbytes,
                                    _lib.stream_ptr(indices.device))
    _lib.check(rc, "stk_b200_pair_plan")
    setattr(indices, _PLAN_ATTR, ((indices._version, offsets.data_ptr(), offsets._version), plan))
    return plan


class DimensionError(AssertionError, ValueError):
    """Incompatible operand sizes (the reference raises AssertionError for these)."""


def _validate_matmul_dims(M, K, N):
    # reference: stk/backend/triton_kernels.py:15-19
    msg = "incompatible dimensions: tensor has dim with length: {}, which must be divisible by {}"
    if M % 128 != 0:
        raise DimensionError(msg.format(M, 128))
    if K % 32 != 0:
        raise DimensionError(msg.format(K, 32))
    if N % 128 != 0:
        raise DimensionError(msg.format(N, 128))


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "stk_b200 matmuls run on CUDA tensors only (there is no CPU path); "
                f"got a tensor on {t.device}")


def _dense_layout(x):
    """(tensor, colmajor, ld) of a 2-D operand the kernels can read in place.

    Row-major (stride (ld, 1)) and exact-transpose views (stride (1, ld)) are consumed as they
    are; anything else, or a misaligned view, is made contiguous first.
    """
    if x.dim() != 2:
        raise DimensionError(f"expected a 2-D dense operand, got {x.dim()}-D")
    rows, cols = x.shape
    s0, s1 = x.stride()
    aligned = x.data_ptr() % 16 == 0
    unit = 16 // x.element_size()          # rows start on 16-byte boundaries
    if s1 == 1 and s0 >= cols and s0 % unit == 0 and aligned:
        return x, 0, s0
    if s0 == 1 and s1 >= rows and s1 % unit == 0 and aligned:
        return x, 1, s1
    x = x.contiguous()
    return x, 0, x.stride(0)


def _check_blocks(data):
    if data.dim() != 3 or data.shape[1] != BLOCK or data.shape[2] != BLOCK:
        raise DimensionError(
            f"block-sparse matmuls need [nnz, {BLOCK}, {BLOCK}] blocks, got {tuple(data.shape)}")
    if not data.is_contiguous():
        raise DimensionError("sparse values must be contiguous")


FP8 = torch.float8_e4m3fn


def _same_dtype(what, *tensors):
    """The kernels read every operand with one element type; mixed float16 / bfloat16 operands would
    be reinterpreted bit for bit.  The last tensors are the outputs: with float8_e4m3fn operands (an
    extension; fp32 accumulation as always) they are bfloat16."""
    dtypes = {t.dtype for t in tensors if t is not None}
    if FP8 in dtypes:
        if dtypes != {FP8, torch.bfloat16}:
            raise ValueError(f"{what}: float8_e4m3fn operands go with each other and a bfloat16 output, got "
                             + ", ".join(sorted(str(d) for d in dtypes)))
        return
    if len(dtypes) > 1:
        raise ValueError(f"{what}: all operands and the output must share one dtype, got "
                         + ", ".join(sorted(str(d) for d in dtypes)))


def dsd(shape, data, offsets, row_indices, column_indices, offsets_t, column_indices_t,
        block_offsets_t, transpose_a, rhs, out):
    """out = op(S) @ rhs, S given by its blocked CSR-COO fields; `shape` is op(S)'s shape."""
    _same_dtype("dsd", data, rhs, out)
    _require_cuda(data, rhs, out)
    if shape[1] != rhs.shape[0]:
        raise DimensionError("incompatible dimensions")
    M, K = shape
    N = rhs.shape[1]
    _validate_matmul_dims(M, K, N)
    _check_blocks(data)
    fp8 = data.dtype == FP8
    rhs, rhs_colmajor, ld_rhs = _dense_layout(rhs)
    if transpose_a:
        meta = (offsets_t, column_indices_t, block_offsets_t)
        pairs = _use_pairs("cols", offsets, row_indices, column_indices, M // BLOCK, offsets_t, column_indices_t)
    else:
        meta = (offsets, column_indices, None)
        pairs = _use_pairs("rows", offsets, row_indices, column_indices, K // BLOCK, offsets_t, column_indices_t)
    if pairs == 0 and N >= 2 * BLOCK and PAIR_MODE in ROW_KERNEL_MODES and not fp8:
        pairs = 3            # one block row x 256 dense columns per CTA
    plan = pair_plan(meta[0], meta[1]) if pairs == 1 else None
    pairs = _pair_shape(pairs, data.shape[0], M // BLOCK, N, out.device)
    with _lib.on_device(out.device):
        rc = _lib.entry("stk_b200_dsd", meta[1])(
            _lib.ptr(data), _lib.ptr(meta[0]), _lib.ptr(meta[1]), _lib.ptr(meta[2]),
            _lib.ptr(rhs), _lib.ptr(out), M, N, K, data.shape[0], int(bool(transpose_a)),
            rhs_colmajor, ld_rhs, out.stride(0), _lib.dtype_code(rhs.dtype), pairs, _lib.ptr(plan),
            _lib.stream_ptr(out.device))
    _lib.check(rc, "stk_b200_dsd")


def dds(lhs, shape, data, offsets, row_indices, column_indices, offsets_t, column_indices_t,
        block_offsets_t, transpose_b, out):
    """out = lhs @ op(S); `shape` is op(S)'s shape."""
    _same_dtype("dds", lhs, data, out)
    _require_cuda(lhs, data, out)
    if lhs.shape[1] != shape[0]:
        raise DimensionError("incompatible dimensions")
    M, K = lhs.shape
    N = shape[1]
    _validate_matmul_dims(M, K, N)
    _check_blocks(data)
    fp8 = data.dtype == FP8
    lhs, lhs_colmajor, ld_lhs = _dense_layout(lhs)
    if transpose_b:
        meta = (offsets, column_indices, None)
        pairs = _use_pairs("rows", offsets, row_indices, column_indices, K // BLOCK, offsets_t, column_indices_t)
    else:
        meta = (offsets_t, column_indices_t, block_offsets_t)
        pairs = _use_pairs("cols", offsets, row_indices, column_indices, N // BLOCK, offsets_t, column_indices_t)
    if pairs == 0 and M >= 2 * BLOCK and PAIR_MODE in ROW_KERNEL_MODES and not fp8:
        pairs = 3            # 256 dense rows x one block column per CTA
    plan = pair_plan(meta[0], meta[1]) if pairs == 1 else None
    pairs = _pair_shape(pairs, data.shape[0], N // BLOCK, M, out.device)
    with _lib.on_device(out.device):
        rc = _lib.entry("stk_b200_dds", meta[1])(
            _lib.ptr(lhs), _lib.ptr(data), _lib.ptr(meta[0]), _lib.ptr(meta[1]), _lib.ptr(meta[2]),
            _lib.ptr(out), M, N, K, data.shape[0], lhs_colmajor, ld_lhs, int(bool(transpose_b)),
            out.stride(0), _lib.dtype_code(lhs.dtype), pairs, _lib.ptr(plan), _lib.stream_ptr(out.device))
    _lib.check(rc, "stk_b200_dds")


def sdd(lhs, rhs, shape, out, offsets, row_indices, column_indices, epilogue=0, aux=None):
    """out[p] = (lhs @ rhs)[block p] for the blocks listed by row_indices / column_indices.
    Extensions: epilogue=1 stores GeLU of the product instead (stk_b200.ops.sdd_gelu); epilogue=2
    stores the product in out and its GeLU in aux; epilogue=3 stores product * GeLU'(aux)
    (stk_b200.dmoe.expert_mlp).  aux has out's shape and dtype."""
    _same_dtype("sdd", lhs, rhs, out, aux)
    _require_cuda(lhs, rhs, out)
    if (epilogue in (2, 3)) != (aux is not None):
        raise ValueError("epilogues 2 and 3 take an auxiliary tensor, the others do not")
    if aux is not None:
        _require_cuda(aux)
        if aux.shape != out.shape or aux.dtype != out.dtype or not aux.is_contiguous():
            raise ValueError("aux must be contiguous with out's shape and dtype")
    if lhs.shape[1] != rhs.shape[0]:
        raise DimensionError("incompatible dimensions")
    M, K = lhs.shape
    N = rhs.shape[1]
    _validate_matmul_dims(M, K, N)
    _check_blocks(out)
    fp8 = lhs.dtype == FP8
    if fp8 and epilogue in (2, 3):
        raise ValueError("the training epilogues are not available with float8 operands")
    lhs, lhs_colmajor, ld_lhs = _dense_layout(lhs)
    rhs, rhs_colmajor, ld_rhs = _dense_layout(rhs)
    pairs = _use_pairs("tiles", offsets, row_indices, column_indices, N // BLOCK)
    if pairs == 0 and not fp8 and (PAIR_MODE == "3" or (PAIR_MODE == "auto" and out.shape[0] >= SDD_ROW_MIN_BLOCKS)):
        pairs = 3            # two blocks of a block row per 128x256 tile
    plan = pair_plan(offsets, column_indices) if pairs == 1 else None
    with _lib.on_device(out.device):
        rc = _lib.entry("stk_b200_sdd", column_indices)(
            _lib.ptr(lhs), _lib.ptr(rhs), _lib.ptr(out), _lib.ptr(offsets), _lib.ptr(row_indices),
            _lib.ptr(column_indices), M, N, K, out.shape[0], lhs_colmajor, ld_lhs, rhs_colmajor,
            ld_rhs, _lib.dtype_code(lhs.dtype), pairs, epilogue, _lib.ptr(aux), _lib.ptr(plan),
            _lib.stream_ptr(out.device))
    _lib.check(rc, "stk_b200_sdd")


def row_indices(shape, data, offsets, column_indices, out):
    """out[p] = block row of block p (CSR offsets -> COO)."""
    _require_cuda(offsets, out)
    if out.dtype not in (torch.int16, torch.int32):
        raise ValueError(f"row indices are int16 or int32, got an output of {out.dtype}")
    block_rows = offsets.numel() - 1
    with _lib.on_device(out.device):
        rc = _lib.entry("stk_b200_row_indices", out)(
            _lib.ptr(offsets), _lib.ptr(out), block_rows, out.numel(), _lib.stream_ptr(out.device))
    _lib.check(rc, "stk_b200_row_indices")


def transpose_meta(row_indices, column_indices, block_cols):
    """(column_indices_t, offsets_t, block_offsets_t) of a topology, on its (CUDA) device."""
    _require_cuda(row_indices, column_indices)
    dev = column_indices.device
    nnz = column_indices.numel()
    if row_indices.dtype != column_indices.dtype:
        raise ValueError("row and column indices must share one integer type")
    column_indices_t = torch.empty(nnz, dtype=column_indices.dtype, device=dev)
    offsets_t = torch.empty(block_cols + 1, dtype=torch.int32, device=dev)
    block_offsets_t = torch.empty(nnz, dtype=torch.int32, device=dev)
    lib = _lib.load()
    ws_bytes = lib.stk_b200_transpose_meta_workspace_bytes(nnz, block_cols)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
    row_indices, column_indices = row_indices.contiguous(), column_indices.contiguous()
    with _lib.on_device(dev):
        rc = _lib.entry("stk_b200_transpose_meta", column_indices)(
            _lib.ptr(row_indices), _lib.ptr(column_indices), nnz,
            block_cols, _lib.ptr(column_indices_t), _lib.ptr(offsets_t), _lib.ptr(block_offsets_t),
            _lib.ptr(ws), ws_bytes, _lib.stream_ptr(dev))
    _lib.check(rc, "stk_b200_transpose_meta")
    return column_indices_t, offsets_t, block_offsets_t


def _elem_bytes(t):
    n = t.element_size()
    if n not in (2, 4) and t.dtype != FP8:
        raise ValueError(f"conversion kernels handle 2- and 4-byte elements and float8_e4m3fn, got {t.dtype}")
    return n


def block_mask(x, blocking):
    """uint8 [R, Cb]: 1 where the blocking x blocking block of x has an element that is not +-0."""
    _require_cuda(x)
    rows, cols = x.shape
    if x.stride(1) != 1:
        x = x.contiguous()
    mask = torch.empty((rows // blocking, cols // blocking), dtype=torch.uint8, device=x.device)
    with _lib.on_device(x.device):
        rc = _lib.load().stk_b200_block_mask(
            _lib.ptr(x), rows, cols, x.stride(0) if rows > 1 else max(cols, 1), blocking,
            _elem_bytes(x), _lib.ptr(mask), _lib.stream_ptr(x.device))
    _lib.check(rc, "stk_b200_block_mask")
    return mask


INT16_BLOCKS = 32767   # most blocks per side that int16 indices can name


def index_dtype_for(block_rows, block_cols):
    """int16 as in the reference (stk/ops/matrix_ops.py:74-75) while it can name every block row and
    column, int32 beyond (the reference raises there, stk/matrix.py:161-167)."""
    return torch.int16 if max(block_rows, block_cols) <= INT16_BLOCKS else torch.int32


def mask_to_topology(mask, index_dtype=None):
    """(offsets, row_indices, column_indices) of a uint8 [R, Cb] block mask (row-major order).

    Reads the block count back to the host to size the index tensors, like torch.nonzero does in
    the reference's to_sparse.  index_dtype: torch.int16 / torch.int32 (default: the narrowest that fits).
    """
    _require_cuda(mask)
    dev = mask.device
    block_rows, block_cols = mask.shape
    mask = mask.contiguous()
    offsets = torch.empty(block_rows + 1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    with _lib.on_device(dev):
        rc = lib.stk_b200_mask_to_offsets(_lib.ptr(mask), block_rows, block_cols, _lib.ptr(offsets),
                                          _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_mask_to_offsets")
        nnz = int(offsets[-1].item())
        if index_dtype is None:
            index_dtype = index_dtype_for(block_rows, block_cols)
        row_idx = torch.empty(nnz, dtype=index_dtype, device=dev)
        col_idx = torch.empty(nnz, dtype=index_dtype, device=dev)
        if nnz == 0:
            return offsets, row_idx, col_idx
        rc = _lib.entry("stk_b200_mask_to_indices", col_idx)(_lib.ptr(mask), block_rows, block_cols, _lib.ptr(offsets),
                                          _lib.ptr(row_idx), _lib.ptr(col_idx), _lib.stream_ptr(dev))
        _lib.check(rc, "stk_b200_mask_to_indices")
    return offsets, row_idx, col_idx


def gather_blocks(x, blocking, row_idx, col_idx, offsets=None):
    """data [nnz, b, b]: the listed blocks of x, copied bit-exactly (offsets: the CSR offsets of the
    list, which let small blocks be copied strip by strip)."""
    _require_cuda(x, row_idx, col_idx)
    rows, cols = x.shape
    if x.stride(1) != 1:
        x = x.contiguous()
    nnz = row_idx.numel()
    data = torch.empty((nnz, blocking, blocking), dtype=x.dtype, device=x.device)
    with _lib.on_device(x.device):
        rc = _lib.entry("stk_b200_gather_blocks", col_idx)(
            _lib.ptr(x), rows, cols, x.stride(0) if rows > 1 else max(cols, 1), blocking,
            _elem_bytes(x), _lib.ptr(offsets), _lib.ptr(row_idx), _lib.ptr(col_idx), nnz, _lib.ptr(data),
            _lib.stream_ptr(x.device))
    _lib.check(rc, "stk_b200_gather_blocks")
    return data


def regroup_blocks(fine, coarse, slot, to_coarse):
    """Moves [nnz, b, b] blocks (b = 16, 32, 64) into (to_coarse) or out of their places inside the
    [n, 128, 128] blocks of `coarse`; slot[p] = coarse block * q*q + (block row % q) * q + block column % q,
    q = 128 // b.  Bit-exact copies; places no block maps to are left as they are."""
    _require_cuda(fine, coarse, slot)
    if fine.dtype != coarse.dtype:
        raise ValueError(f"regroup_blocks: one dtype for both sides, got {fine.dtype} and {coarse.dtype}")
    if fine.dim() != 3 or fine.shape[1] != fine.shape[2] or coarse.dim() != 3 or tuple(coarse.shape[1:]) != (BLOCK, BLOCK):
        raise DimensionError(f"regroup_blocks: expected [nnz, b, b] and [n, {BLOCK}, {BLOCK}] blocks, got "
                             f"{tuple(fine.shape)} and {tuple(coarse.shape)}")
    if not fine.is_contiguous() or not coarse.is_contiguous() or slot.dtype != torch.int32 or slot.numel() != fine.shape[0]:
        raise DimensionError("regroup_blocks: contiguous blocks and one int32 slot per block")
    with _lib.on_device(fine.device):
        rc = _lib.load().stk_b200_regroup_blocks(
            _lib.ptr(fine) if fine.numel() else None, _lib.ptr(coarse) if coarse.numel() else None,
            _lib.ptr(slot) if slot.numel() else None, fine.shape[0], coarse.shape[0], fine.shape[1],
            _elem_bytes(fine), int(bool(to_coarse)), _lib.stream_ptr(fine.device))
    _lib.check(rc, "stk_b200_regroup_blocks")


def to_dense(data, offsets, column_indices, block_rows, block_cols, blocking):
    """Dense [R*b, Cb*b] tensor with the blocks in place and zeros elsewhere."""
    _require_cuda(data, offsets, column_indices)
    out = torch.empty((block_rows * blocking, block_cols * blocking), dtype=data.dtype,
                      device=data.device)
    if out.numel() == 0:
        return out
    data = data.contiguous()
    with _lib.on_device(data.device):
        rc = _lib.entry("stk_b200_to_dense", column_indices)(
            _lib.ptr(data) if data.numel() else None, _lib.ptr(offsets),
            _lib.ptr(column_indices) if column_indices.numel() else None, block_rows, block_cols,
            blocking, _elem_bytes(data), _lib.ptr(out), out.stride(0), _lib.stream_ptr(data.device))
    _lib.check(rc, "stk_b200_to_dense")
    return out
