"""stk.ops.dsd / dds / sdd: block-sparse products (reference: stk/ops/linear_ops.py:7-59).

S = sparse (stk.Matrix), D = dense (torch.Tensor); the three letters are output, left, right.
"""
import torch

from stk_b200.backend import sputnik
from stk_b200.matrix import Matrix


def _fields(m):
    return (m.data, m.offsets, m.row_indices, m.column_indices, m.offsets_t, m.column_indices_t,
            m.block_offsets_t)


def dsd(a, b):
    """dense = a @ b with a sparse (possibly a .t() view) and b dense."""
    assert isinstance(a, Matrix)
    assert isinstance(b, torch.Tensor)
    return sputnik.dsd(a.size(), *_fields(a), not a.is_contiguous(), b)


def dds(a, b):
    """dense = a @ b with a dense and b sparse (possibly a .t() view)."""
    assert isinstance(a, torch.Tensor)
    assert isinstance(b, Matrix)
    return sputnik.dds(a, b.size(), *_fields(b), not b.is_contiguous())


def sdd(a, b, topo):
    """sparse = (a @ b) evaluated only on the nonzero blocks of `topo`."""
    assert isinstance(a, torch.Tensor)
    assert isinstance(b, torch.Tensor)
    assert isinstance(topo, Matrix)
    assert topo.is_contiguous()
    out = sputnik.sdd(a, b, topo.size(), *_fields(topo))
    return Matrix(topo.size(), out, topo.row_indices, topo.column_indices, topo.offsets,
                  topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)


@torch.no_grad()
def sdd_gelu(a, b, topo):
    """sparse = GeLU(a @ b) on the nonzero blocks of `topo`, the activation applied to the fp32
    accumulator inside the matmul kernel (torch.nn.functional.gelu's exact form).

    An extension over the reference API: the sdd -> GeLU -> dsd step of a dMoE layer writes its
    hidden activations once instead of write / read / write.  Forward only (not differentiable);
    training code uses sdd followed by gelu on Matrix.data."""
    from stk_b200.backend import kernels
    assert isinstance(a, torch.Tensor)
    assert isinstance(b, torch.Tensor)
    assert isinstance(topo, Matrix)
    assert topo.is_contiguous()
    out = torch.empty(topo.data.shape, dtype=a.dtype, device=a.device)
    kernels.sdd(a, b, topo.size(), out, topo.offsets, topo.row_indices, topo.column_indices,
                epilogue=1)
    return Matrix(topo.size(), out, topo.row_indices, topo.column_indices, topo.offsets,
                  topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
