"""Generates the golden fixtures in this directory by running the REFERENCE itself.

Run from the repository root, in a container that has the reference checkout:

    TRITON_INTERPRET=1 PYTHONPATH=<reference root> python tests/golden/make_golden.py

* metadata.npz  - stk.random.mask (dense mask -> to_sparse -> Matrix -> _transpose) on CPU tensors
* convert.npz   - stk.ops.to_sparse / to_dense on seeded dense inputs, special values included
* matmul.npz    - stk.ops.sdd / dsd / dds forward results of the reference's Triton kernels, executed
                  by the Triton interpreter on CPU tensors (no GPU involved)

The Triton interpreter cannot execute bfloat16 kernels (numpy has no such type and the results are
garbage), so the bf16 cases run the reference kernels on float32 copies of the bf16 operands - every
bf16 value is exact in float32 and the kernels accumulate in float32 either way - and the float32
result is rounded to bf16 with torch (round to nearest even, the rounding of the kernels' final cast).

Inputs are not stored: they are regenerated from oracle.stk_oracle.hash_tensor and numpy seeds.
16-bit float tensors are stored as their raw uint16 bit patterns.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

import stk  # noqa: E402  (the reference)

from oracle import stk_oracle as oracle  # noqa: E402
from tests import cases  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def fields(m, prefix):
    return {
        f"{prefix}/row_indices": m.row_indices.numpy(),
        f"{prefix}/column_indices": m.column_indices.numpy(),
        f"{prefix}/offsets": m.offsets.numpy(),
        f"{prefix}/column_indices_t": m.column_indices_t.numpy(),
        f"{prefix}/offsets_t": m.offsets_t.numpy(),
        f"{prefix}/block_offsets_t": m.block_offsets_t.numpy(),
    }


def make_metadata():
    out = {}
    for name, (rows, cols, sparsity, blocking, seed) in cases.METADATA_CASES.items():
        np.random.seed(seed)
        m = stk.random.mask(rows, cols, sparsity, blocking)
        m.validate()
        out.update(fields(m, name))
        out[f"{name}/data_shape"] = np.array(m.data.shape)
        assert bool((m.data == 1).all())
    np.savez_compressed(os.path.join(HERE, "metadata.npz"), **out)
    print("metadata.npz:", len(cases.METADATA_CASES), "cases")


def make_convert():
    out = {}
    for name in cases.CONVERT_CASES:
        x = cases.convert_input(name)
        rows, cols, sparsity, blocking, seed, dtype = cases.CONVERT_CASES[name]
        m = stk.ops.to_sparse(x, blocking)
        out.update(fields(m, name))
        out[f"{name}/data_bits"] = bits(m.data)
        out[f"{name}/data_shape"] = np.array(m.data.shape)
        dense = stk.ops.to_dense(m)
        # the reference's own round-trip property (matrix_ops_test.py:26-58); NaN breaks == so
        # compare bits, ignoring the sign of zeros in dropped blocks
        assert dense.shape == x.shape
        out[f"{name}/dense_bits"] = bits(dense)
    np.savez_compressed(os.path.join(HERE, "convert.npz"), **out)
    print("convert.npz:", len(cases.CONVERT_CASES), "cases")


def make_matmul():
    out = {}
    for name in cases.MATMUL_CASES:
        op, trans_a, trans_b, dtype = cases.MATMUL_CASES[name]
        inp = cases.matmul_inputs(name)
        run_dtype = torch.float32 if dtype == torch.bfloat16 else dtype
        for key in ("a", "b", "data", "dense"):
            if key in inp:
                inp[key] = inp[key].to(run_dtype)
        if op == "sdd":
            topo = stk.Matrix(inp["topo_shape"], torch.empty(len(inp["row_indices"]), 128, 128, dtype=run_dtype),
                              torch.from_numpy(inp["row_indices"]), torch.from_numpy(inp["column_indices"]),
                              torch.from_numpy(inp["offsets"]))
            a = inp["a"].t() if trans_a else inp["a"]
            b = inp["b"].t() if trans_b else inp["b"]
            res = stk.ops.sdd(a, b, topo).data
        else:
            s = stk.Matrix(inp["sparse_shape"], inp["data"], torch.from_numpy(inp["row_indices"]),
                           torch.from_numpy(inp["column_indices"]), torch.from_numpy(inp["offsets"]))
            if op == "dsd":
                a = s.t() if trans_a else s
                b = inp["dense"].t() if trans_b else inp["dense"]
                res = stk.ops.dsd(a, b)
            else:
                a = inp["dense"].t() if trans_a else inp["dense"]
                b = s.t() if trans_b else s
                res = stk.ops.dds(a, b)
        out[f"{name}/out_bits"] = bits(res.to(dtype))
        out[f"{name}/out_shape"] = np.array(res.shape)
        print(name, tuple(res.shape))
    np.savez_compressed(os.path.join(HERE, "matmul.npz"), **out)


if __name__ == "__main__":
    make_metadata()
    make_convert()
    make_matmul()
