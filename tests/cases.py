"""Seeded inputs shared by the golden-fixture generator, the oracle tests and the GPU parity tests.

Everything here is regenerated from seeds (numpy's global RNG for block patterns, exactly as the
reference draws them, and oracle.stk_oracle.hash_tensor for values), so fixtures only hold outputs.
"""
import numpy as np
import torch

from oracle import stk_oracle as oracle

# name -> (rows, cols, sparsity, blocking, numpy seed) for stk.random.mask.
# The first fifteen are the reference's own conversion / random test cases
# (stk/ops/matrix_ops_test.py:8-23, stk/random/random_ops_test.py:8-23); "c1" is the benchmark's
# CPU-runnable configuration, the rest add 128-blocking topologies with ties in every column.
METADATA_CASES = {
    "t00": (8, 16, 0.0, 1, 0), "t01": (8, 16, 0.5, 1, 1), "t02": (8, 16, 0.95, 1, 2),
    "t03": (16, 8, 0.0, 1, 3), "t04": (16, 8, 0.5, 1, 4), "t05": (16, 8, 0.95, 1, 5),
    "t06": (8, 16, 0.0, 8, 6), "t07": (8, 16, 0.5, 8, 7), "t08": (8, 16, 1.0, 8, 8),
    "t09": (16, 8, 0.0, 8, 9), "t10": (16, 8, 0.5, 8, 10), "t11": (16, 8, 1.0, 8, 11),
    "t12": (128, 256, 0.5, 16, 12), "t13": (256, 128, 0.75, 32, 13), "t14": (512, 512, 0.875, 128, 14),
    "c1": (1024, 1024, 0.75, 128, 0),
    "wide": (1024, 4096, 0.5, 128, 21),
    "tall": (4096, 1024, 0.8, 128, 22),
    "dense": (1024, 1024, 0.0, 128, 23),
    "sq205": (2048, 2048, 0.2, 128, 24),
    "big": (6144, 6144, 0.5, 128, 25),
}

# name -> (rows, cols, sparsity, blocking, seed, dtype)
CONVERT_CASES = {
    "b1": (8, 16, 0.5, 1, 31, torch.float16),
    "b8": (16, 8, 0.5, 8, 32, torch.float16),
    "b16": (128, 256, 0.5, 16, 33, torch.float16),
    "b32": (256, 128, 0.75, 32, 34, torch.float16),
    "b128": (512, 512, 0.875, 128, 35, torch.float16),
    "b128_bf16": (384, 512, 0.5, 128, 36, torch.bfloat16),
    "special": (256, 384, 0.0, 128, 37, torch.float16),
    "empty": (256, 256, 1.0, 128, 38, torch.float16),
}


def convert_input(name):
    rows, cols, sparsity, blocking, seed, dtype = CONVERT_CASES[name]
    np.random.seed(seed)
    mask = oracle.dense_mask(rows, cols, sparsity, blocking)
    x = (oracle.hash_tensor((rows, cols), seed, 1.0, torch.float32) * mask).to(dtype)
    if name == "special":
        # 2 x 3 blocks: all +0 | all -0 | one NaN
        #               one Inf | one denormal | one -0 among +0 (still empty)
        x.zero_()
        x[:128, 128:256] = -0.0
        x[5, 300] = float("nan")
        x[200, 7] = float("inf")
        x[130, 129] = 6e-8  # fp16 denormal
        x[129, 257] = -0.0
    return x


# name -> (op, trans_a, trans_b, dtype); sizes in matmul_inputs
def _matmul_cases():
    out = {}
    for op in ("sdd", "dsd", "dds"):
        for ta in (False, True):
            for tb in (False, True):
                tag = ("t" if ta else "n") + ("t" if tb else "n")
                out[f"{op}_{tag}_f16"] = (op, ta, tb, torch.float16)
                if ta == tb:
                    out[f"{op}_{tag}_bf16"] = (op, ta, tb, torch.bfloat16)
    return out


MATMUL_CASES = _matmul_cases()

_SPARSE_ROWS, _SPARSE_COLS = 384, 256  # 3 x 2 blocks
_SDD_K = 160                            # a multiple of 32 that is not a multiple of 64
_DENSE_DIM = 128


def _topology(rows, cols, seed):
    np.random.seed(seed)
    pat = oracle.block_pattern(rows, cols, 0.5, 128)
    r, c = np.nonzero(pat)
    offsets = np.concatenate([[0], np.cumsum(pat.sum(axis=1))]).astype(np.int32)
    return r.astype(np.int16), c.astype(np.int16), offsets


def matmul_inputs(name):
    """Operands of a golden matmul case, in STORAGE layout (transposes are applied as views,
    as in stk/ops/linear_ops_test.py:72-75,88-91)."""
    op, trans_a, trans_b, dtype = MATMUL_CASES[name]
    seed = sorted(MATMUL_CASES).index(name) + 100
    if op == "sdd":
        m, n, k = _SPARSE_ROWS, _SPARSE_COLS, _SDD_K
        r, c, offsets = _topology(m, n, seed)
        a = oracle.hash_tensor((k, m) if trans_a else (m, k), seed, 0.1, dtype)
        b = oracle.hash_tensor((n, k) if trans_b else (k, n), seed + 1000, 0.1, dtype)
        return dict(a=a, b=b, row_indices=r, column_indices=c, offsets=offsets,
                    topo_shape=torch.Size((m, n)))
    # The sparse operand is stored [384, 256]; used as is or transposed.
    r, c, offsets = _topology(_SPARSE_ROWS, _SPARSE_COLS, seed)
    data = oracle.hash_tensor((len(r), 128, 128), seed, 0.1, dtype)
    trans_sparse = trans_a if op == "dsd" else trans_b
    trans_dense = trans_b if op == "dsd" else trans_a
    s_rows, s_cols = (_SPARSE_COLS, _SPARSE_ROWS) if trans_sparse else (_SPARSE_ROWS, _SPARSE_COLS)
    if op == "dsd":   # [s_rows, s_cols] @ [s_cols, 128]
        logical = (s_cols, _DENSE_DIM)
    else:             # [128, s_rows] @ [s_rows, s_cols]
        logical = (_DENSE_DIM, s_rows)
    stored = (logical[1], logical[0]) if trans_dense else logical
    dense = oracle.hash_tensor(stored, seed + 1000, 0.1, dtype)
    return dict(data=data, dense=dense, row_indices=r, column_indices=c, offsets=offsets,
                sparse_shape=torch.Size((_SPARSE_ROWS, _SPARSE_COLS)))
