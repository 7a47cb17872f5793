"""Autograd functions DSD, DDS, SDD and RowIndices over the sm_100a kernel launchers.

The module keeps the name, the function signatures and the saved state of the reference's glue
layer (stk/backend/sputnik.py: DSD :85-158, DDS :161-231, SDD :234-302, RowIndices :304-316) so that
stk.ops.linear_ops can call it unchanged.  The backward passes are written from the calculus
rather than from the reference's transpose tables:

    C = op(A) @ op(B)
    d op(A) = dC @ op(B)^T          d op(B) = op(A)^T @ dC

and a gradient wanted in the storage layout of a transposed operand is the transpose of that
product, i.e. the product of the transposed factors in reverse order.  A product lands in SDD, DSD
or DDS depending on which of (left factor, right factor, result) is sparse.  As in the reference,
the gradient of a dense operand that came in as an exact ``.t()`` view is computed in the view's
storage layout and returned as a ``.t()`` view.
"""
import torch

from stk_b200.backend import kernels as backend
from stk_b200.backend.autocast import custom_bwd, custom_fwd


def _is_transposed(x):
    """True for an exact ``.t()`` view of a contiguous 2-D tensor."""
    return (not x.is_contiguous() and x.stride()[0] == 1 and x.stride()[1] == x.size()[0])


class _SparseOperand:
    """A sparse factor of a product: logical shape, the seven fields and a transposed flag."""

    __slots__ = ("shape", "data", "meta", "transposed")

    def __init__(self, shape, data, meta, transposed):
        self.shape = torch.Size(shape)  # logical shape of op(S)
        self.data = data
        self.meta = meta  # (offsets, row_indices, column_indices, offsets_t, column_indices_t, block_offsets_t)
        self.transposed = transposed

    def t(self):
        return _SparseOperand((self.shape[1], self.shape[0]), self.data, self.meta,
                              not self.transposed)

    @property
    def storage_shape(self):
        return torch.Size((self.shape[1], self.shape[0])) if self.transposed else self.shape


def _matmul(a, b, topology=None):
    """a @ b through the autograd functions; `topology` selects the sparse-output product."""
    if topology is not None:
        return sdd(a, b, topology.storage_shape, topology.data, *topology.meta)
    if isinstance(a, _SparseOperand):
        return dsd(a.shape, a.data, *a.meta, a.transposed, b)
    return dds(a, b.shape, b.data, *b.meta, b.transposed)


def _grad_of_dense(left, right, operand):
    """Gradient left @ right of the dense tensor `operand`, laid out like `operand`."""
    if _is_transposed(operand):
        return _matmul(right.t(), left.t()).t()
    return _matmul(left, right)


def _grad_of_sparse(left, right, topology):
    """Values of (left @ right) on `topology`, in the storage layout of its blocks."""
    if topology.transposed:
        return _matmul(right.t(), left.t(), topology)
    return _matmul(left, right, topology)


def _tidy(dy):
    """Gradients arrive with arbitrary strides; keep row-major and exact-transpose layouts."""
    if not dy.is_contiguous() and not _is_transposed(dy):
        return dy.contiguous()
    return dy


class DSD(torch.autograd.Function):
    """out = op(S) @ rhs."""

    @staticmethod
    @custom_fwd
    def forward(ctx, shape, data, offsets, row_indices, column_indices, offsets_t,
                column_indices_t, block_offsets_t, transpose_a, rhs):
        ctx.save_for_backward(data, offsets, row_indices, column_indices, offsets_t,
                              column_indices_t, block_offsets_t, rhs)
        ctx.shape = torch.Size(shape)  # logical shape of op(S)
        ctx.transpose_a = transpose_a
        out = torch.empty((shape[0], rhs.size()[1]), dtype=rhs.dtype, device=rhs.device)
        backend.dsd(shape, data, offsets, row_indices, column_indices, offsets_t,
                    column_indices_t, block_offsets_t, transpose_a, rhs, out)
        return out

    @staticmethod
    @custom_bwd
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        sparse = _SparseOperand(ctx.shape, saved[0], tuple(saved[1:7]), ctx.transpose_a)
        rhs = saved[7]
        dy = _tidy(dy)
        ddata = drhs = None
        if ctx.needs_input_grad[1]:
            ddata = _grad_of_sparse(dy, rhs.t(), sparse)
        if ctx.needs_input_grad[9]:
            drhs = _grad_of_dense(sparse.t(), dy, rhs)
        return None, ddata, None, None, None, None, None, None, None, drhs


dsd = DSD.apply


class DDS(torch.autograd.Function):
    """out = lhs @ op(S)."""

    @staticmethod
    @custom_fwd
    def forward(ctx, lhs, shape, data, offsets, row_indices, column_indices, offsets_t,
                column_indices_t, block_offsets_t, transpose_b):
        ctx.save_for_backward(lhs, data, offsets, row_indices, column_indices, offsets_t,
                              column_indices_t, block_offsets_t)
        ctx.shape = torch.Size(shape)
        ctx.transpose_b = transpose_b
        out = torch.empty((lhs.size()[0], shape[1]), dtype=lhs.dtype, device=lhs.device)
        backend.dds(lhs, shape, data, offsets, row_indices, column_indices, offsets_t,
                    column_indices_t, block_offsets_t, transpose_b, out)
        return out

    @staticmethod
    @custom_bwd
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        lhs = saved[0]
        sparse = _SparseOperand(ctx.shape, saved[1], tuple(saved[2:8]), ctx.transpose_b)
        dy = _tidy(dy)
        dlhs = ddata = None
        if ctx.needs_input_grad[0]:
            dlhs = _grad_of_dense(dy, sparse.t(), lhs)
        if ctx.needs_input_grad[2]:
            ddata = _grad_of_sparse(lhs.t(), dy, sparse)
        return dlhs, None, ddata, None, None, None, None, None, None, None


dds = DDS.apply


class SDD(torch.autograd.Function):
    """out = (lhs @ rhs) sampled on a block topology; `data` only donates the output shape."""

    @staticmethod
    @custom_fwd
    def forward(ctx, lhs, rhs, shape, data, offsets, row_indices, column_indices, offsets_t,
                column_indices_t, block_offsets_t):
        ctx.save_for_backward(lhs, rhs, offsets, row_indices, column_indices, offsets_t,
                              column_indices_t, block_offsets_t)
        ctx.shape = torch.Size(shape)
        out = torch.empty(data.shape, dtype=lhs.dtype, device=lhs.device)
        backend.sdd(lhs, rhs, shape, out, offsets, row_indices, column_indices)
        return out

    @staticmethod
    @custom_bwd
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        lhs, rhs = saved[0], saved[1]
        if not dy.is_contiguous():
            dy = dy.contiguous()
        grad = _SparseOperand(ctx.shape, dy, tuple(saved[2:8]), False)
        dlhs = drhs = None
        if ctx.needs_input_grad[0]:
            dlhs = _grad_of_dense(grad, rhs.t(), lhs)
        if ctx.needs_input_grad[1]:
            drhs = _grad_of_dense(lhs.t(), grad, rhs)
        return dlhs, drhs, None, None, None, None, None, None, None, None


sdd = SDD.apply


class RowIndices(torch.autograd.Function):
    """Block-row index of every block, from the CSR offsets."""

    @staticmethod
    def forward(ctx, shape, data, offsets, column_indices):
        out = torch.empty(column_indices.shape, dtype=column_indices.dtype,
                          device=column_indices.device)
        backend.row_indices(shape, data, offsets, column_indices, out)
        return out


row_indices = RowIndices.apply
