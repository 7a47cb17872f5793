"""stk.ops.mul (reference: stk/ops/eltwise_ops.py:3-28)."""
from stk_b200.matrix import Matrix


def mul(a, b):
    """Element-wise product of two sparse matrices that share a's topology.

    The caller guarantees that b has the same topology as a; the result reuses a's metadata.
    """
    assert isinstance(a, Matrix)
    assert isinstance(b, Matrix)
    assert a.size() == b.size()
    return Matrix(a.size(), a.data * b.data, a.row_indices, a.column_indices, a.offsets,
                  a.column_indices_t, a.offsets_t, a.block_offsets_t)
