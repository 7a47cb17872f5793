"""stk.ops.to_sparse / to_dense / ones_like / row_indices / sum
(reference: stk/ops/matrix_ops.py:7-98).

The reference expands an int64 index for every nonzero ELEMENT and uses scatter_/gather; here each
conversion is a handful of block-level kernels (see stk_b200.backend.kernels).  Results are
bit-identical: the same blocks in the same order, values copied untouched.
"""
import numpy as np
import torch

from stk_b200.backend import kernels as _kernels
from stk_b200.backend import sputnik
from stk_b200.matrix import Matrix, compute_device


@torch.no_grad()
def row_indices(shape, data, offsets, column_indices):
    return sputnik.row_indices(shape, data, offsets, column_indices)


@torch.no_grad()
def to_dense(x):
    """Dense tensor of x's shape.

    For a transposed view the reference scatters the storage layout into the transposed shape
    (stk/ops/matrix_ops.py:39-47), which is not the transpose; here a transposed view gives the
    transposed dense matrix.
    """
    assert isinstance(x, Matrix)
    if not x.is_contiguous():
        return to_dense(x.t()).t().contiguous()
    shape = (int(np.prod(x.shape[:-1])), int(x.shape[-1]))
    b = x.blocking
    home = x.device
    dev = compute_device(x.data)
    out = _kernels.to_dense(x.data.to(dev), x.offsets.to(dev), x.column_indices.to(dev),
                            shape[0] // b, shape[1] // b, b)
    return out.to(home).reshape(x.size())


@torch.no_grad()
def _mask(x, blocking=1):
    """bool [R, Cb]: which blocks of the 2-D tensor x hold a nonzero."""
    assert x.dim() == 2
    assert x.size()[0] % blocking == 0
    assert x.size()[1] % blocking == 0
    dev = compute_device(x)
    return _kernels.block_mask(x.to(dev), blocking).to(x.device) != 0


@torch.no_grad()
def to_sparse(x, blocking=1, index_dtype=None):
    """Blocked CSR-COO form of the 2-D tensor x; blocks that are entirely +-0 are dropped.
    index_dtype (not in the reference): torch.int16 or torch.int32 for the block indices; by default
    int16 as in the reference, int32 when x has more than 32767 blocks per side."""
    assert x.dim() == 2
    assert x.size()[0] % blocking == 0
    assert x.size()[1] % blocking == 0
    home = x.device
    dev = compute_device(x)
    xd = x.to(dev)
    mask = _kernels.block_mask(xd, blocking)
    offsets, row_idx, col_idx = _kernels.mask_to_topology(mask, index_dtype)
    data = _kernels.gather_blocks(xd, blocking, row_idx, col_idx, offsets)
    col_t, off_t, blk_t = _kernels.transpose_meta(row_idx, col_idx, x.size()[1] // blocking)
    fields = [t.to(home) for t in (data, row_idx, col_idx, offsets, col_t, off_t, blk_t)]
    return Matrix(x.size(), *fields)


@torch.no_grad()
def ones_like(x):
    return Matrix(x.size(), torch.ones_like(x.data), x.row_indices, x.column_indices, x.offsets,
                  x.column_indices_t, x.offsets_t, x.block_offsets_t)


def sum(x):
    assert isinstance(x, Matrix)
    return x.data.sum()
