"""stk.Matrix: a block-sparse matrix in blocked CSR-COO form.

Same constructor, properties and methods as the reference class (stk/matrix.py:126-329); the
transpose metadata that the reference derives with argsort / gather / histc / cumsum
(stk/matrix.py:105-123) comes from the stable counting-sort kernel behind
stk_b200.backend.kernels.transpose_meta.  Within one block column the reference's default
(unstable) argsort leaves the order of the blocks unspecified; here it is always ascending block
row, which is what a stable sort gives.
"""
import numpy as np
import torch

from stk_b200.backend import kernels as _kernels

_INT16_MAX = int(np.iinfo(np.int16).max)


def compute_device(t):
    """Device the kernels run on for tensor `t`: its own if CUDA, else the current CUDA device.

    Host tensors are staged through the GPU (the reference runs the same steps as torch CPU ops;
    this package has no CPU implementation to fall back to).
    """
    if t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise RuntimeError(
            "stk_b200 has no CPU path: this operation runs CUDA kernels and needs a CUDA device")
    return torch.device("cuda", torch.cuda.current_device())


def _validate_matrix(shape, data, row_indices, column_indices, offsets):
    """Shape / dtype / device checks of the five defining fields (stk/matrix.py:14-102).

    Returns `data` viewed as [nnz, block, block].  Unlike the reference, bfloat16 values are
    accepted next to float16 (its matmuls are tested with both), and the block indices may be int32
    instead of int16 (needed beyond 32767 blocks per side).
    """
    if data.dim() == 1:
        data = data.reshape(data.numel(), 1, 1)
    if data.shape[-2] != data.shape[-1]:
        raise ValueError("Expected square blocking in data. "
                         f"Got block shape {[data.shape[-2], data.shape[-1]]}")
    block = data.shape[-1]
    data = data.view(-1, block, block)
    if shape[-2] % block != 0 or shape[-1] % block != 0:
        raise ValueError("Matrix shape must be dividible by blocking. "
                         f"Got shape {tuple(shape)} with {[block, block]} blocking.")
    if np.prod(shape) < data.numel():
        raise ValueError("Invalid matrix. Number of nonzeros exceeds matrix capacity "
                         f"({data.numel()} v. {np.prod(shape)})")
    for name, t in (("row_indices", row_indices), ("column_indices", column_indices),
                    ("offsets", offsets)):
        if t.dim() != 1:
            raise ValueError(f"Expected 1D {name}. Got {t.dim()}D {name}.")
    for name, t in (("row_indices", row_indices), ("column_indices", column_indices)):
        if t.numel() != data.shape[0]:
            raise ValueError("Expected 1 index per nonzero block. "
                             f"Got {t.numel()} {name} for {data.shape[0]} blocks")
    block_rows = np.prod(shape[:-1]) / block
    if offsets.numel() != block_rows + 1:
        raise ValueError("Expected one offset per block row plus one. "
                         f"Got {offsets.numel()} offsets with {block_rows} block rows.")
    devices = {t.is_cuda for t in (data, row_indices, column_indices, offsets)}
    if len(devices) != 1:
        raise ValueError("Expected data & meta-data on common device. "
                         f"Got data on {data.device}, row_indices on {row_indices.device} "
                         f"column_indices on {column_indices.device} and "
                         f"offsets on {offsets.device}.")
    if data.dtype not in (torch.float16, torch.bfloat16, torch.float8_e4m3fn):
        raise ValueError(f"Expected float16, bfloat16 or float8_e4m3fn data. Got {data.dtype} data.")
    for name, t in (("row_indices", row_indices), ("column_indices", column_indices)):
        if t.dtype not in (torch.int16, torch.int32):
            raise ValueError(f"Expected int16 or int32 {name}. Got {t.dtype} {name}.")
    if row_indices.dtype != column_indices.dtype:
        raise ValueError("Expected row_indices and column_indices of one integer type. "
                         f"Got {row_indices.dtype} and {column_indices.dtype}.")
    if offsets.dtype != torch.int32:
        raise ValueError(f"Expected int32 offsets. Got {offsets.dtype} offsets.")
    return data


def _transpose(size, data, row_indices, column_indices, offsets):
    """(column_indices_t, offsets_t, block_offsets_t) for the given topology."""
    block_columns = size[1] // data.shape[1]
    home = column_indices.device
    dev = compute_device(column_indices)
    out = _kernels.transpose_meta(row_indices.to(dev), column_indices.to(dev), block_columns)
    return tuple(t.to(home) for t in out)


class Matrix(torch.nn.Module):
    """A matrix stored in block compressed sparse row form with COO row indices.

    Fields (dtypes as produced by stk.ops.to_sparse): data [nnz, b, b]; row_indices and
    column_indices int16 [nnz]; offsets int32 [block_rows + 1]; and the same topology in
    column-major order: column_indices_t int16 [nnz] (block rows), offsets_t int32
    [block_cols + 1], block_offsets_t int32 [nnz] (positions in data).  A matrix with more than 32767
    blocks per side carries int32 row_indices / column_indices / column_indices_t instead (the
    reference rejects such sizes, stk/matrix.py:161-167).
    """

    def __init__(self, size, data, row_indices, column_indices, offsets, column_indices_t=None,
                 offsets_t=None, block_offsets_t=None):
        super().__init__()
        self._size = size
        self._data = data
        self._row_indices = row_indices
        self._column_indices = column_indices
        self._offsets = offsets
        if column_indices_t is None or offsets_t is None or block_offsets_t is None:
            column_indices_t, offsets_t, block_offsets_t = _transpose(
                size, data, row_indices, column_indices, offsets)
        self._column_indices_t = column_indices_t
        self._offsets_t = offsets_t
        self._block_offsets_t = block_offsets_t
        self._transposed = False

        # 16-bit block indices bound the representable size.
        if column_indices.dtype == torch.int16:
            limit = _INT16_MAX * self.blocking
            if size[0] > limit or size[1] > limit:
                raise ValueError(f"Sparse matrix with shape {tuple(size)} exceeds representable "
                                 "size with 16-bit indices.")

    def _like(self, size, data):
        """A Matrix over `data` that shares this one's metadata tensors."""
        return Matrix(size, data, self._row_indices, self._column_indices, self._offsets,
                      self._column_indices_t, self._offsets_t, self._block_offsets_t)

    def validate(self):
        _validate_matrix(self._size, self._data, self._row_indices, self._column_indices,
                         self._offsets)

    def to(self, device):
        """Moves every tensor to `device` (reference: stk/matrix.py:178-185).  A floating dtype (an
        extension; the reference leaves it as a TODO) converts the values only - the metadata keeps
        its integer types."""
        if isinstance(device, torch.dtype):
            if device not in (torch.float16, torch.bfloat16, torch.float8_e4m3fn):
                raise ValueError(f"Expected float16, bfloat16 or float8_e4m3fn data. Got {device}.")
            self._data = self._data.to(device)
            return self
        for name in ("_data", "_row_indices", "_column_indices", "_offsets", "_column_indices_t",
                     "_offsets_t", "_block_offsets_t"):
            setattr(self, name, getattr(self, name).to(device))
        return self

    def cuda(self):
        return self.to(torch.cuda.current_device())

    def clone(self):
        return Matrix(self.size(), self.data.clone(), self.row_indices.clone(),
                      self.column_indices.clone(), self.offsets.clone(),
                      self.column_indices_t.clone(), self.offsets_t.clone(),
                      self.block_offsets_t.clone())

    def t(self):
        """O(1) transposed view: shares every tensor; the kernels read the *_t metadata."""
        if self.dim() != 2:
            raise ValueError("t() expects a tensor with <= 2 dimensions, "
                             f"but self is {self.dim()}D.")
        out = self._like(self.size(), self.data)
        out._transposed = not self._transposed
        out._size = torch.Size((self._size[1], self._size[0]))
        return out

    def contiguous(self):
        raise ValueError("Not yet implemented.")

    def is_contiguous(self):
        return not self._transposed

    @property
    def is_cuda(self):
        return self._data.is_cuda

    @property
    def device(self):
        return self._data.device

    def size(self):
        return self._size

    @property
    def shape(self):
        return self.size()

    def dim(self):
        return len(self._size)

    @property
    def data(self):
        return self._data

    @property
    def row_indices(self):
        return self._row_indices

    @property
    def column_indices(self):
        return self._column_indices

    @property
    def offsets(self):
        return self._offsets

    @property
    def offsets_t(self):
        return self._offsets_t

    @property
    def column_indices_t(self):
        return self._column_indices_t

    @property
    def block_offsets_t(self):
        return self._block_offsets_t

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def nnz(self):
        return self.data.numel()

    @property
    def blocking(self):
        return self.data.shape[1]

    @property
    def requires_grad(self):
        return self.data.requires_grad

    def requires_grad_(self, x):
        self.data.requires_grad_(x)
        return self

    def view(self, *shape):
        assert self.is_contiguous()
        if shape[-1] != self.size()[-1]:
            raise ValueError("Can't change view on compressed dimension. "
                             f"{self.size()[-1]} v. {shape[-1]}.")
        if np.prod(shape) != np.prod(self.size()):
            raise ValueError("Mismatch in numel of Matrix and new shape. "
                             f"{np.prod(self.size())} v. {np.prod(shape)}")
        return self._like(shape, self.data)

    @property
    def grad(self):
        """The gradient of the values, wrapped with this matrix's topology (and orientation)."""
        size = self.size()
        if not self.is_contiguous():
            size = torch.Size((size[1], size[0]))
        out = self._like(size, self.data.grad)
        return out if self.is_contiguous() else out.t()
