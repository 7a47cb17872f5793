"""Products of matrices whose blocks are 16, 32 or 64 wide.

The reference has matmul kernels for 128 x 128 blocks only (stk/backend/triton_kernels.py:8-11: BLOCK_SIZE
is fixed at 128) although its Matrix and conversions take any blocking.  Here a matrix with smaller blocks
takes part in sdd / dsd / dds as the matrix of the 128 x 128 blocks that contain its blocks, zero where it
has none:

    dsd / dds: the values are copied into zero-filled 128-blocks, then the 128-block product runs; the
               added zeros contribute exact zeros to every fp32 sum.
    sdd:       the product is sampled on the containing 128-blocks, then the b x b blocks of the topology
               are copied out of them; every kept element is the same fp32 sum, rounded once.

The containing topology (unique 128-blocks, their CSR and transposed metadata, and the place of every small
block inside them) is computed once per topology and cached on its column_indices tensor.  The copies are one
kernel (stk_b200_regroup_blocks) and are differentiable: the backward of a copy into the 128-blocks is the
copy out of them and the other way round, so gradients of the small-block values come out of the 128-block
backward passes unchanged.  Cost: up to (128 / b)^2 times the MMA work of a native b x b kernel when no two
small blocks share a 128-block, none when they tile it.
"""
import torch

from stk_b200.backend import kernels
from stk_b200.matrix import Matrix

BLOCK = kernels.BLOCK
SMALL_BLOCKINGS = (16, 32, 64)
_ATTR = "_stk_b200_coarse_topology"


class _Coarse:
    """The 128-block topology containing a small-block topology (storage orientation)."""

    __slots__ = ("size", "fields", "blocks", "slot")

    def __init__(self, size, fields, blocks, slot):
        self.size = size          # storage shape (rows, cols)
        self.fields = fields      # row_indices, column_indices, offsets, column_indices_t, offsets_t, block_offsets_t
        self.blocks = blocks      # number of 128-blocks
        self.slot = slot          # int32 [nnz]: place of every small block (see stk_b200_regroup_blocks)

    def matrix(self, data):
        return Matrix(self.size, data, *self.fields)

    def placeholder(self, dtype, device):
        """A [blocks, 128, 128] tensor without storage behind it: sdd reads only its shape and dtype."""
        return torch.empty(1, dtype=dtype, device=device).expand(self.blocks, BLOCK, BLOCK)


def _storage_size(m):
    rows, cols = m.size()
    return (rows, cols) if m.is_contiguous() else (cols, rows)


def coarse_topology(m):
    """_Coarse of Matrix `m` (any orientation; computed for the storage orientation and cached)."""
    b = m.blocking
    if b not in SMALL_BLOCKINGS:
        raise kernels.DimensionError(
            f"block-sparse matmuls take blocks of {BLOCK} or of {SMALL_BLOCKINGS}, got {b}")
    if m.dim() != 2:
        raise kernels.DimensionError(f"expected a 2-D sparse matrix, got {m.dim()}-D")
    rows, cols = _storage_size(m)
    if rows % BLOCK or cols % BLOCK:
        raise kernels.DimensionError(
            f"incompatible dimensions: a sparse matrix of shape {(rows, cols)} must be divisible by {BLOCK}")
    col_idx, row_idx = m.column_indices, m.row_indices
    stamp = (col_idx._version, row_idx.data_ptr(), row_idx._version, b, rows, cols)
    cached = getattr(col_idx, _ATTR, None)
    if cached is not None and cached[0] == stamp:
        return cached[1]
    q = BLOCK // b
    block_rows, block_cols = rows // BLOCK, cols // BLOCK
    r, c = row_idx.long(), col_idx.long()
    key = (r // q) * block_cols + c // q
    uniq, inverse = torch.unique(key, sorted=True, return_inverse=True)    # reads the count back: once per topology
    crow, ccol = uniq // block_cols, uniq % block_cols
    offsets = torch.zeros(block_rows + 1, dtype=torch.int32, device=col_idx.device)
    if uniq.numel():
        offsets[1:] = torch.cumsum(torch.bincount(crow, minlength=block_rows), 0)
    slot = (inverse * (q * q) + (r % q) * q + c % q).to(torch.int32)
    index_dtype = col_idx.dtype
    first = Matrix((rows, cols), torch.empty(1, dtype=m.dtype, device=m.device).expand(uniq.numel(), BLOCK, BLOCK),
                   crow.to(index_dtype), ccol.to(index_dtype), offsets)
    coarse = _Coarse((rows, cols),
                     (first.row_indices, first.column_indices, first.offsets, first.column_indices_t,
                      first.offsets_t, first.block_offsets_t), int(uniq.numel()), slot)
    setattr(col_idx, _ATTR, (stamp, coarse))
    return coarse


class _Regroup(torch.autograd.Function):
    """values -> the same values in the other blocking (into zero-filled 128-blocks, or out of 128-blocks)."""

    @staticmethod
    def forward(ctx, values, slot, coarse_blocks, blocking, to_coarse):
        ctx.save_for_backward(slot)
        ctx.args = (coarse_blocks, blocking, to_coarse)
        return _regroup(values, slot, coarse_blocks, blocking, to_coarse)

    @staticmethod
    def backward(ctx, grad):
        coarse_blocks, blocking, to_coarse = ctx.args
        return _regroup(grad, ctx.saved_tensors[0], coarse_blocks, blocking, not to_coarse), None, None, None, None


def _regroup(values, slot, coarse_blocks, blocking, to_coarse):
    values = values.contiguous()
    if to_coarse:
        q = BLOCK // blocking
        # every small block has its own place, so as many blocks as places means no place is left to zero
        make = torch.empty if slot.numel() == coarse_blocks * q * q else torch.zeros
        out = make((coarse_blocks, BLOCK, BLOCK), dtype=values.dtype, device=values.device)
        kernels.regroup_blocks(values, out, slot, True)
    else:
        out = torch.empty((slot.numel(), blocking, blocking), dtype=values.dtype, device=values.device)
        kernels.regroup_blocks(out, values, slot, False)
    return out


def as_blocks_of_128(m):
    """Matrix with 128-blocks holding the values of `m` (same orientation), differentiable in m.data."""
    coarse = coarse_topology(m)
    out = coarse.matrix(_Regroup.apply(m.data, coarse.slot, coarse.blocks, m.blocking, True))
    return out if m.is_contiguous() else out.t()


def topology_of_128(topo, dtype):
    """The containing 128-block topology of `topo` as a Matrix for sdd (no values behind it)."""
    coarse = coarse_topology(topo)
    return coarse.matrix(coarse.placeholder(dtype, topo.device)), coarse


def from_blocks_of_128(product, coarse, topo):
    """The blocks of `topo` out of an sdd result on its containing topology."""
    data = _Regroup.apply(product.data, coarse.slot, coarse.blocks, topo.blocking, False)
    return Matrix(topo.size(), data, topo.row_indices, topo.column_indices, topo.offsets,
                  topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
