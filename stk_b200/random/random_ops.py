"""stk.random.dense_mask / mask / randn (reference: stk/random/random_ops.py:6-36).

The block pattern is drawn with the same numpy call on the same global RNG as the reference, so a
seeded run gives the same topology.  `mask` then builds the sparse matrix straight from the
block-level pattern instead of tiling it to a dense element-level fp16 matrix first.
"""
import numpy as np
import torch

from stk_b200.backend import kernels as _kernels
from stk_b200.matrix import Matrix, compute_device


def _block_pattern(rows, cols, sparsity, blocking):
    """float64 [R, Cb] of ones with round(R*Cb*sparsity-ish) entries zeroed, as in the reference."""
    assert sparsity >= 0.0 and sparsity <= 1.0
    assert rows % blocking == 0 and cols % blocking == 0
    block_rows, block_cols = rows // blocking, cols // blocking
    nnz = round(block_rows * block_cols * (1 - sparsity))
    out = np.ones(block_rows * block_cols)
    zeroed = np.random.choice(out.size, out.size - nnz, replace=False)
    out[zeroed] = 0.0
    return out.reshape(block_rows, block_cols)


@torch.no_grad()
def dense_mask(rows, cols, sparsity, blocking=1):
    """float32 [rows, cols] 0/1 mask whose blocking x blocking blocks are all-0 or all-1."""
    pattern = torch.from_numpy(_block_pattern(rows, cols, sparsity, blocking).astype(np.float32))
    return pattern.repeat_interleave(blocking, dim=0).repeat_interleave(blocking, dim=1)


@torch.no_grad()
def mask(m, n, sparsity, blocking=1):
    """Sparse fp16 matrix of ones with a random block pattern (lives on the host, like the
    reference's)."""
    pattern = torch.from_numpy(_block_pattern(m, n, sparsity, blocking).astype(np.uint8))
    dev = compute_device(pattern)
    offsets, row_idx, col_idx = _kernels.mask_to_topology(pattern.to(dev))
    col_t, off_t, blk_t = _kernels.transpose_meta(row_idx, col_idx, n // blocking)
    data = torch.ones((row_idx.numel(), blocking, blocking), dtype=torch.float16)
    meta = [t.cpu() for t in (row_idx, col_idx, offsets, col_t, off_t, blk_t)]
    return Matrix(torch.Size((m, n)), data, *meta)


@torch.no_grad()
def randn(shape, sparsity, blocking=1):
    shape_2d = (int(np.prod(shape[:-1])), shape[-1])
    out = mask(*shape_2d, sparsity, blocking)
    out.data.copy_(torch.randn(*out.data.shape))
    return out.view(*shape)
