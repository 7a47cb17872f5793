"""stk_b200: the Sparse Toolkit API (stk.Matrix, stk.ops, stk.random) on B200-native kernels.

    import stk_b200 as stk

is a drop-in for ``import stk``.  The block-sparse products and the metadata / conversion steps run
as hand-written sm_100a CUDA kernels loaded from libstk_b200.so through its C ABI
(include/stk_b200.h); there is no Triton and no CPU fallback.
"""
import stk_b200.random
import stk_b200.ops
from stk_b200.matrix import Matrix

__all__ = ["Matrix", "ops", "random"]
