"""The reference's linear-op test matrix (stk/ops/linear_ops_test.py:21-213): 14 sizes x 4 transpose
combinations x {fp16, bf16}, forward and both gradients of dsd, dds and sdd.

The expected values are the dense fp32 products of the same 16-bit inputs (torch on the GPU, as in
the reference's tests), compared with this repository's parity tolerance, which is tighter than the
reference's (rtol 5e-2 with 0.25 % outliers allowed)."""
import itertools

import pytest
import torch

from tests.parity import assert_product_close

pytestmark = pytest.mark.gpu

_MATRIX_SIZES = (
    (128, 128, 128, 0.0), (256, 256, 256, 0.5), (2048, 1024, 512, 0.8), (512, 128, 128, 0.0),
    (128, 128, 512, 0.0), (1024, 512, 512, 0.0), (1024, 512, 512, 0.5), (1024, 512, 512, 0.75),
    (512, 512, 1024, 0.0), (512, 512, 1024, 0.5), (512, 512, 1024, 0.75), (1024, 1024, 1024, 0.0),
    (1024, 1024, 1024, 0.5), (1024, 1024, 1024, 0.75),
)
_TRANSPOSE = ((False, False), (False, True), (True, False), (True, True))
_DTYPE = (torch.float16, torch.bfloat16)
_CASES = [(*size, *trans, dtype)
          for size, trans, dtype in itertools.product(_MATRIX_SIZES, _TRANSPOSE, _DTYPE)]
_IDS = [f"{m}x{k}x{n}-s{s}-{'t' if ta else 'n'}{'t' if tb else 'n'}-{str(dt)[6:]}"
        for m, k, n, s, ta, tb, dt in _CASES]


@pytest.fixture(scope="module", params=["0", "1", "2", "3"], ids=["tile128", "pair256", "wide512", "row256"])
def stk(request):
    """The package with the matmul kernel choice forced: one 128x128 tile per CTA, or 256x256
    supertiles on CTA pairs (both must give the same results on every topology)."""
    import stk_b200
    from stk_b200.backend import kernels, lib
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = request.param
    yield stk_b200
    kernels.PAIR_MODE = saved
    assert lib.device_status() == 0


def _dense_and_sparse(stk, rows, cols, sparsity, dtype, std=0.1):
    mask = stk.random.dense_mask(rows, cols, sparsity, 128)
    dense = (torch.randn(rows, cols) * std * mask).type(dtype).cuda()
    sparse = stk.ops.to_sparse(dense, 128)
    return dense.float().requires_grad_(True), sparse.requires_grad_(True)


def _dense(rows, cols, dtype, std=0.1):
    x = (torch.randn(rows, cols) * std).type(dtype).cuda()
    return x.requires_grad_(True), x.detach().float().requires_grad_(True)


def _t(x, flag):
    return x.t() if flag else x


def _mask_of(stk, m):
    return stk.ops.to_dense(stk.ops.ones_like(m)).float()


@pytest.mark.parametrize("m,k,n,sparsity,trans_a,trans_b,dtype", _CASES, ids=_IDS)
def test_dsd(stk, m, k, n, sparsity, trans_a, trans_b, dtype):
    torch.manual_seed(m + k + n)
    a_dense, a = _dense_and_sparse(stk, *((k, m) if trans_a else (m, k)), sparsity, dtype)
    b, b32 = _dense(*((n, k) if trans_b else (k, n)), dtype)
    out = stk.ops.dsd(_t(a, trans_a), _t(b, trans_b))
    expected = torch.mm(_t(a_dense, trans_a), _t(b32, trans_b))
    expected.sum().backward()
    out.sum().backward()
    assert out.dtype == dtype
    assert_product_close(out, expected, "dsd forward")
    assert_product_close(stk.ops.to_dense(a.grad), a_dense.grad * _mask_of(stk, a.grad), "dsd dlhs")
    assert b.grad.shape == b.shape
    assert_product_close(b.grad, b32.grad, "dsd drhs")


@pytest.mark.parametrize("m,k,n,sparsity,trans_a,trans_b,dtype", _CASES, ids=_IDS)
def test_dds(stk, m, k, n, sparsity, trans_a, trans_b, dtype):
    torch.manual_seed(m + k + n + 1)
    a, a32 = _dense(*((k, m) if trans_a else (m, k)), dtype)
    b_dense, b = _dense_and_sparse(stk, *((n, k) if trans_b else (k, n)), sparsity, dtype)
    out = stk.ops.dds(_t(a, trans_a), _t(b, trans_b))
    expected = torch.mm(_t(a32, trans_a), _t(b_dense, trans_b))
    expected.sum().backward()
    out.sum().backward()
    assert out.dtype == dtype
    assert_product_close(out, expected, "dds forward")
    assert a.grad.shape == a.shape
    assert_product_close(a.grad, a32.grad, "dds dlhs")
    assert_product_close(stk.ops.to_dense(b.grad), b_dense.grad * _mask_of(stk, b.grad), "dds drhs")


@pytest.mark.parametrize("m,k,n,sparsity,trans_a,trans_b,dtype", _CASES, ids=_IDS)
def test_sdd(stk, m, k, n, sparsity, trans_a, trans_b, dtype):
    torch.manual_seed(m + k + n + 2)
    a, a32 = _dense(*((k, m) if trans_a else (m, k)), dtype)
    b, b32 = _dense(*((n, k) if trans_b else (k, n)), dtype)
    _, topo = _dense_and_sparse(stk, m, n, sparsity, dtype)
    mask = _mask_of(stk, topo)
    out = stk.ops.sdd(_t(a, trans_a), _t(b, trans_b), topo)
    expected = torch.mm(_t(a32, trans_a), _t(b32, trans_b)) * mask
    expected.sum().backward()
    stk.ops.sum(out).backward()
    assert out.dtype == dtype
    assert_product_close(stk.ops.to_dense(out), expected, "sdd forward")
    assert_product_close(a.grad, a32.grad, "sdd dlhs")
    assert_product_close(b.grad, b32.grad, "sdd drhs")
