"""CPU restatement of the reference's block-sparse matmul path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may import
this module, and only as the checker or the timed CPU baseline; nothing in stk_b200/ does.

Parity status: PINNED.  tests/golden/ holds outputs of the reference itself (its torch-op metadata
and conversion routines run on CPU, and its Triton kernels run under TRITON_INTERPRET=1), produced
by tests/golden/make_golden.py; tests/test_oracle.py checks every function below against them.

Integer work is numpy; floating-point products use torch CPU matmul in fp32, which is what the
reference's own tests compare against (stk/ops/linear_ops_test.py:83-96).  File:line citations
are relative to the reference project root.
"""
import numpy as np
import torch


# ---------------------------------------------------------------------------- metadata
def row_indices(offsets):
    """CSR offsets -> block-row index per block, int16.
    Follows _row_indices_kernel, stk/backend/triton_kernels.py:381-387: block row `pid` writes
    `pid` into out[offsets[pid] : offsets[pid+1]]."""
    offsets = np.asarray(offsets, dtype=np.int64)
    counts = np.diff(offsets)
    return np.repeat(np.arange(len(counts), dtype=np.int16), counts)


def transpose(block_cols, row_idx, col_idx):
    """(column_indices_t int16, offsets_t int32, block_offsets_t int32).
    Follows _transpose, stk/matrix.py:105-123: argsort of column_indices (:110), gather of
    row_indices (:111), the permutation itself as int32 (:112), histogram + cumsum of the column
    indices for offsets_t (:117-122).  The reference's argsort is the default unstable one, which
    leaves the order inside one column unspecified; this restatement fixes it to the stable order
    (ascending storage index, hence ascending block row)."""
    row_idx = np.asarray(row_idx, dtype=np.int16)
    col_idx = np.asarray(col_idx, dtype=np.int16)
    perm = np.argsort(col_idx, kind="stable")
    column_indices_t = row_idx[perm].astype(np.int16)
    block_offsets_t = perm.astype(np.int32)
    counts = np.bincount(col_idx.astype(np.int64), minlength=block_cols)[:block_cols]
    offsets_t = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return column_indices_t, offsets_t, block_offsets_t


def canonical_tie_order(column_indices_t, offsets_t, block_offsets_t):
    """Sort every column segment of a reference result by block_offsets_t, which maps any valid
    tie order of the reference's unstable argsort onto the stable one."""
    cit = np.array(column_indices_t).copy()
    bot = np.array(block_offsets_t).copy()
    for c in range(len(offsets_t) - 1):
        lo, hi = int(offsets_t[c]), int(offsets_t[c + 1])
        order = np.argsort(bot[lo:hi], kind="stable")
        cit[lo:hi] = cit[lo:hi][order]
        bot[lo:hi] = bot[lo:hi][order]
    return cit, bot


def block_mask(x, blocking):
    """bool [R, Cb]: block kept iff sum(|x|) over it != 0.
    Follows _mask, stk/ops/matrix_ops.py:50-59.  The sum of absolute values is nonzero exactly
    when some element is not +-0 (NaN and Inf included), which is how it is evaluated here — on
    the raw bits, so that bf16 needs no float conversion."""
    bits = _bits(x)
    rows, cols = bits.shape
    absbits = bits & (np.iinfo(bits.dtype).max >> 1 if bits.dtype.kind == "u" else 0)
    nz = absbits != 0
    return nz.reshape(rows // blocking, blocking, cols // blocking, blocking).any(axis=(1, 3))


def to_sparse(x, blocking):
    """dict with data (same dtype as x, [nnz,b,b]), row_indices, column_indices, offsets and the
    transposed metadata.  Follows to_sparse, stk/ops/matrix_ops.py:64-85: row counts -> offsets
    (:68-71), nonzero(mask) in row-major order -> int16 indices (:73-75), gather of the blocks'
    elements (:78-84), then Matrix() -> _transpose (:85)."""
    m = block_mask(x, blocking)
    rows, cols = x.shape
    offsets = np.concatenate([[0], np.cumsum(m.sum(axis=1))]).astype(np.int32)
    r, c = np.nonzero(m)
    r16, c16 = r.astype(np.int16), c.astype(np.int16)
    xt = x if isinstance(x, torch.Tensor) else torch.from_numpy(np.asarray(x))
    blocks = xt.reshape(rows // blocking, blocking, cols // blocking, blocking).permute(0, 2, 1, 3)
    data = blocks[torch.from_numpy(r), torch.from_numpy(c)].contiguous()
    cit, offt, bot = transpose(cols // blocking, r16, c16)
    return dict(data=data, row_indices=r16, column_indices=c16, offsets=offsets,
                column_indices_t=cit, offsets_t=offt, block_offsets_t=bot)


def to_dense(data, row_idx, col_idx, shape):
    """Dense torch tensor with block p at (row_idx[p]*b, col_idx[p]*b), zeros elsewhere.
    Follows to_dense, stk/ops/matrix_ops.py:36-47 (zeros + scatter of every block element)."""
    data = data if isinstance(data, torch.Tensor) else torch.from_numpy(np.asarray(data))
    b = data.shape[1] if data.dim() == 3 else 1
    rows, cols = int(shape[0]), int(shape[1])
    out = torch.zeros(rows // b, cols // b, b, b, dtype=data.dtype)
    if data.shape[0]:
        out[torch.from_numpy(np.asarray(row_idx, dtype=np.int64)),
            torch.from_numpy(np.asarray(col_idx, dtype=np.int64))] = data
    return out.permute(0, 2, 1, 3).reshape(rows, cols).contiguous()


def block_pattern(rows, cols, sparsity, blocking):
    """float64 [R, Cb] 0/1 pattern drawn from numpy's global RNG.
    Follows dense_mask, stk/random/random_ops.py:8-16: nnz = round(R*Cb*(1-sparsity)) (Python
    rounding), then np.random.choice(R*Cb, R*Cb-nnz, replace=False) positions are zeroed."""
    block_rows, block_cols = rows // blocking, cols // blocking
    nnz = round(block_rows * block_cols * (1 - sparsity))
    out = np.ones(block_rows * block_cols)
    out[np.random.choice(out.size, out.size - nnz, replace=False)] = 0.0
    return out.reshape(block_rows, block_cols)


def dense_mask(rows, cols, sparsity, blocking):
    """float32 [rows, cols]; follows stk/random/random_ops.py:18-22 (np.tile to element level)."""
    pat = block_pattern(rows, cols, sparsity, blocking)
    return torch.from_numpy(np.kron(pat, np.ones((blocking, blocking))).astype(np.float32))


def mask(rows, cols, sparsity, blocking):
    """to_sparse of the fp16 dense mask; follows stk/random/random_ops.py:26-28."""
    return to_sparse(dense_mask(rows, cols, sparsity, blocking).to(torch.float16), blocking)


# ---------------------------------------------------------------------------- products
def _f32(x):
    return x.to(torch.float32)


def sdd(lhs, rhs, row_idx, col_idx, out_dtype, blocking=128):
    """[nnz,b,b] values of lhs @ rhs on the listed blocks, fp32 accumulation, rounded to out_dtype.
    Follows the reference tests' oracle _mmm, stk/ops/linear_ops_test.py:83-85 (torch.mm times the
    topology's dense mask), restricted to the kept blocks; per block it is what _sdd_kernel
    computes, stk/backend/triton_kernels.py:44-68."""
    full = _f32(lhs) @ _f32(rhs)
    b = blocking
    blocks = full.reshape(full.shape[0] // b, b, full.shape[1] // b, b).permute(0, 2, 1, 3)
    out = blocks[torch.from_numpy(np.asarray(row_idx, dtype=np.int64)),
                 torch.from_numpy(np.asarray(col_idx, dtype=np.int64))]
    return out.to(out_dtype).contiguous()


def dsd(sparse_dense, rhs, out_dtype):
    """op(S) @ rhs with op(S) given densified (to_dense, transposed if needed); fp32 accumulate.
    Follows testLinearOps_Dsd's expected value, stk/ops/linear_ops_test.py:102-112, and
    _dsd_kernel, stk/backend/triton_kernels.py:101-145."""
    return (_f32(sparse_dense) @ _f32(rhs)).to(out_dtype)


def dds(lhs, sparse_dense, out_dtype):
    """lhs @ op(S); follows stk/ops/linear_ops_test.py:139-149 and _dds_kernel,
    stk/backend/triton_kernels.py:178-220."""
    return (_f32(lhs) @ _f32(sparse_dense)).to(out_dtype)


def reference_cpu_path_sdd(lhs, rhs, data, row_idx, col_idx, shape):
    """The reference's own CPU-runnable formulation, in the operand dtype:
    torch.mm(a, b) * to_dense(ones_like(topo)), stk/ops/linear_ops_test.py:83-85.
    This is the timed CPU baseline."""
    mask_dense = to_dense(torch.ones_like(data), row_idx, col_idx, shape)
    return torch.mm(lhs, rhs) * mask_dense


def reference_cpu_path_dsd(data, row_idx, col_idx, shape, rhs):
    """to_dense(S) then torch.mm, stk/ops/linear_ops_test.py:104-112.  Timed CPU baseline."""
    return torch.mm(to_dense(data, row_idx, col_idx, shape), rhs)


# ---------------------------------------------------------------------------- helpers
def _bits(x):
    """Raw bit pattern of a 2-/4-byte tensor or array as an unsigned numpy array."""
    if isinstance(x, torch.Tensor):
        if x.element_size() == 2:
            return x.contiguous().view(torch.int16).numpy().view(np.uint16)
        return x.contiguous().view(torch.int32).numpy().view(np.uint32)
    x = np.ascontiguousarray(x)
    return x.view(np.uint16 if x.itemsize == 2 else np.uint32)


def rel_rms_error(out, ref):
    """max |out - ref| / RMS(ref), both taken to fp32 — the parity metric of the matmuls."""
    out, ref = _f32(out), _f32(ref)
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-30)
    return ((out - ref).abs().max() / rms).item()


def hash_tensor(shape, seed, scale, dtype):
    """Deterministic pseudo-random tensor that depends on no library's RNG stream, so golden
    inputs can be regenerated anywhere: splitmix64 of (seed, index) -> uniform(-1, 1) * scale."""
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        z = np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        z += np.full(n, seed + 1, dtype=np.uint64) * np.uint64(0xD1B54A32D192ED03)
        z ^= z >> np.uint64(30)
        z *= np.uint64(0xBF58476D1CE4E5B9)
        z ^= z >> np.uint64(27)
        z *= np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    unit = (z >> np.uint64(40)).astype(np.float64) / float(1 << 24)  # [0, 1)
    out = torch.from_numpy(((unit * 2.0 - 1.0) * scale).astype(np.float32).reshape(shape))
    return out.to(dtype)
