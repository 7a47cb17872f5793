"""stk.ops.dsd / dds / sdd: block-sparse products (reference: stk/ops/linear_ops.py:7-59).

S = sparse (stk.Matrix), D = dense (torch.Tensor); the three letters are output, left, right.
"""
import torch

from stk_b200.backend import kernels, sputnik
from stk_b200.matrix import Matrix
from stk_b200.ops import small_blocks


def _fields(m):
    return (m.data, m.offsets, m.row_indices, m.column_indices, m.offsets_t, m.column_indices_t,
            m.block_offsets_t)


# float8_e4m3fn operands (not in the reference): fp32 accumulation, bfloat16 result, forward only; the
# same operand layouts and .t() views as with 16-bit operands.
def _is_fp8(*tensors):
    return any(t.dtype == kernels.FP8 for t in tensors)


def _no_grad_fp8(*tensors):
    if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
        raise ValueError("float8 products are forward only; call them under torch.no_grad()")


def dsd(a, b, out=None):
    """dense = a @ b with a sparse (possibly a .t() view) and b dense.

    `out` (not in the reference): a row-major [rows of a, columns of b] tensor of b's dtype to write
    the product into instead of a fresh one, e.g. a buffer other GPUs read.  No gradient flows
    through a product written this way, and autocast does not apply to it.
    """
    assert isinstance(a, Matrix)
    assert isinstance(b, torch.Tensor)
    if a.blocking in small_blocks.SMALL_BLOCKINGS:      # 16-, 32-, 64-blocks run inside the 128-blocks that contain them
        return dsd(small_blocks.as_blocks_of_128(a), b, out)
    if out is None and _is_fp8(a.data, b):
        _no_grad_fp8(a.data, b)
        out = torch.empty((a.size()[0], b.shape[1]), dtype=torch.bfloat16, device=b.device)
        kernels.dsd(a.size(), *_fields(a), not a.is_contiguous(), b, out)
        return out
    if out is None:
        return sputnik.dsd(a.size(), *_fields(a), not a.is_contiguous(), b)
    if torch.is_grad_enabled() and (a.data.requires_grad or b.requires_grad):
        raise ValueError("dsd(out=...) does not record a gradient; call it under torch.no_grad()")
    want = torch.bfloat16 if _is_fp8(a.data, b) else b.dtype
    if (out.dim() != 2 or out.shape[0] != a.size()[0] or out.shape[1] != b.shape[1] or out.dtype != want
            or out.stride(1) != 1 or out.device != b.device):
        raise ValueError("out must be a row-major [a.size(0), b.size(1)] tensor of b's dtype (bfloat16 for "
                         "float8 operands) on b's device")
    kernels.dsd(a.size(), *_fields(a), not a.is_contiguous(), b, out)
    return out


def dds(a, b):
    """dense = a @ b with a dense and b sparse (possibly a .t() view)."""
    assert isinstance(a, torch.Tensor)
    assert isinstance(b, Matrix)
    if b.blocking in small_blocks.SMALL_BLOCKINGS:
        return dds(a, small_blocks.as_blocks_of_128(b))
    if _is_fp8(a, b.data):
        _no_grad_fp8(a, b.data)
        out = torch.empty((a.shape[0], b.size()[1]), dtype=torch.bfloat16, device=a.device)
        kernels.dds(a, b.size(), *_fields(b), not b.is_contiguous(), out)
        return out
    return sputnik.dds(a, b.size(), *_fields(b), not b.is_contiguous())


def sdd(a, b, topo):
    """sparse = (a @ b) evaluated only on the nonzero blocks of `topo`."""
    assert isinstance(a, torch.Tensor)
    assert isinstance(b, torch.Tensor)
    assert isinstance(topo, Matrix)
    assert topo.is_contiguous()
    if topo.blocking in small_blocks.SMALL_BLOCKINGS:
        containing, coarse = small_blocks.topology_of_128(topo, a.dtype)
        return small_blocks.from_blocks_of_128(sdd(a, b, containing), coarse, topo)
    if _is_fp8(a, b):
        _no_grad_fp8(a, b)
        out = torch.empty(topo.data.shape, dtype=torch.bfloat16, device=a.device)
        kernels.sdd(a, b, topo.size(), out, topo.offsets, topo.row_indices, topo.column_indices)
    else:
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
    if topo.blocking in small_blocks.SMALL_BLOCKINGS:
        containing, coarse = small_blocks.topology_of_128(topo, a.dtype)
        return small_blocks.from_blocks_of_128(sdd_gelu(a, b, containing), coarse, topo)
    out = torch.empty(topo.data.shape, dtype=torch.bfloat16 if _is_fp8(a, b) else a.dtype, device=a.device)
    kernels.sdd(a, b, topo.size(), out, topo.offsets, topo.row_indices, topo.column_indices,
                epilogue=1)
    return Matrix(topo.size(), out, topo.row_indices, topo.column_indices, topo.offsets,
                  topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
