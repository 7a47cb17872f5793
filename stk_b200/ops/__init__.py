from stk_b200.ops.linear_ops import dds, dsd, sdd, sdd_gelu
from stk_b200.ops.matrix_ops import ones_like, row_indices, sum, to_dense, to_sparse
from stk_b200.ops.eltwise_ops import mul
