"""Products of matrices with 16-, 32- and 64-blocks (the reference's matmuls exist for 128-blocks only,
stk/backend/triton_kernels.py:8-11; its Matrix and conversions take any blocking): against the oracle,
against the dense autograd path for the gradients, and the copy kernel bit for bit."""
import numpy as np
import pytest
import torch

from oracle import stk_oracle as oracle
from tests.parity import assert_product_close, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["0", "auto"], ids=["tile128", "auto"])
def stk(request):
    import stk_b200
    from stk_b200.backend import kernels, lib
    assert torch.cuda.is_available()
    lib.load()
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = request.param
    yield stk_b200
    kernels.PAIR_MODE = saved
    assert lib.device_status() == 0


def _topology(stk, rows, cols, sparsity, blocking, seed):
    np.random.seed(seed)
    torch.manual_seed(seed)
    return stk.random.mask(rows, cols, sparsity, blocking)


@pytest.mark.parametrize("blocking", [16, 32, 64])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_products_with_small_blocks_match_the_oracle(stk, blocking, dtype):
    rows, cols, inner = 512, 384, 256
    topo = _topology(stk, rows, cols, 0.7, blocking, blocking)
    r, c = topo.row_indices.numpy(), topo.column_indices.numpy()
    nnz = len(r)
    assert nnz > 0
    g = torch.Generator().manual_seed(7)
    a = (torch.randn(rows, inner, generator=g) * 0.05).to(dtype)
    b = (torch.randn(inner, cols, generator=g) * 0.05).to(dtype)
    topo_d = topo.to("cuda").to(dtype)
    for ta in (False, True):
        for tb in (False, True):
            A = a.t().contiguous().cuda().t() if ta else a.cuda()
            B = b.t().contiguous().cuda().t() if tb else b.cuda()
            out = stk.ops.sdd(A, B, topo_d)
            assert out.blocking == blocking and out.data.shape == (nnz, blocking, blocking)
            assert_product_close(out.data, oracle.sdd(a, b, r, c, dtype, blocking), f"sdd {ta}{tb}")
    vals = (torch.randn(nnz, blocking, blocking, generator=g) * 0.05).to(dtype)
    s = stk.Matrix(topo.size(), vals.cuda(), topo_d.row_indices, topo_d.column_indices, topo_d.offsets,
                   topo_d.column_indices_t, topo_d.offsets_t, topo_d.block_offsets_t)
    s_dense = oracle.to_dense(vals, r, c, (rows, cols))
    right = (torch.randn(cols, inner, generator=g) * 0.05).to(dtype)
    right_t = (torch.randn(rows, inner, generator=g) * 0.05).to(dtype)
    assert_product_close(stk.ops.dsd(s, right.cuda()), oracle.dsd(s_dense, right, dtype), "dsd")
    assert_product_close(stk.ops.dsd(s.t(), right_t.cuda()), oracle.dsd(s_dense.t(), right_t, dtype), "dsd T")
    assert_product_close(stk.ops.dsd(s, right.t().contiguous().cuda().t()), oracle.dsd(s_dense, right, dtype),
                         "dsd, column-major dense")
    assert_product_close(stk.ops.dds(right_t.t().cuda(), s), oracle.dds(right_t.t(), s_dense, dtype), "dds")
    assert_product_close(stk.ops.dds(right.t().cuda(), s.t()), oracle.dds(right.t(), s_dense.t(), dtype), "dds T")
    # the fused activation (exact erf form of the fp32 sums) on the kept blocks
    fused = stk.ops.sdd_gelu(a.cuda(), b.cuda(), topo_d)
    keep = oracle.to_dense(torch.ones(nnz, blocking, blocking), r, c, (rows, cols))
    want = (torch.nn.functional.gelu(a.float() @ b.float()) * keep).to(dtype)
    assert_product_close(stk.ops.to_dense(fused), want, "sdd_gelu")


@pytest.mark.parametrize("blocking", [32, 64])
def test_small_block_sdd_is_the_128_block_sdd_sampled(stk, blocking):
    """Every kept element is the fp32 sum the 128-block kernel forms, rounded once: bit-identical to the
    same elements of an sdd over all 128-blocks."""
    rows = cols = 512
    topo = _topology(stk, rows, cols, 0.6, blocking, 3).to("cuda")
    everything = _topology(stk, rows, cols, 0.0, 128, 0).to("cuda")
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(rows, 192, generator=g) * 0.1).half().cuda()
    b = (torch.randn(192, cols, generator=g) * 0.1).half().cuda()
    small = stk.ops.to_dense(stk.ops.sdd(a, b, topo))
    full = stk.ops.to_dense(stk.ops.sdd(a, b, everything))
    kept = stk.ops.to_dense(stk.Matrix(topo.size(), torch.ones_like(topo.data), topo.row_indices, topo.column_indices,
                                       topo.offsets, topo.column_indices_t, topo.offsets_t, topo.block_offsets_t))
    np.testing.assert_array_equal(bits(small), bits(torch.where(kept != 0, full, torch.zeros_like(full))))


@pytest.mark.parametrize("blocking", [16, 64])
def test_gradients_with_small_blocks_match_dense_autograd(stk, blocking):
    rows, cols, inner = 256, 384, 128
    topo = _topology(stk, rows, cols, 0.5, blocking, 11).to("cuda")
    r, c = topo.row_indices.cpu().numpy(), topo.column_indices.cpu().numpy()
    nnz = len(r)
    g = torch.Generator().manual_seed(5)
    vals = (torch.randn(nnz, blocking, blocking, generator=g) * 0.1).half()
    dense_rhs = (torch.randn(cols, inner, generator=g) * 0.1).half()
    lhs = (torch.randn(rows, inner, generator=g) * 0.1).half()
    # dsd: gradients of the sparse values and of the dense operand
    s = stk.Matrix(topo.size(), vals.cuda().requires_grad_(True), topo.row_indices, topo.column_indices,
                   topo.offsets, topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
    d = dense_rhs.cuda().requires_grad_(True)
    out = stk.ops.dsd(s, d)
    dy = (torch.randn(rows, inner, generator=g) * 0.1).half()
    out.backward(dy.cuda())
    v32 = vals.float().requires_grad_(True)
    d32 = dense_rhs.float().requires_grad_(True)
    keep = oracle.to_dense(torch.ones(nnz, blocking, blocking), r, c, (rows, cols))
    index = (torch.from_numpy(r.astype(np.int64)), torch.from_numpy(c.astype(np.int64)))

    def densify(v):
        grid = torch.zeros(rows // blocking, cols // blocking, blocking, blocking)
        grid = grid.index_put(index, v)
        return grid.permute(0, 2, 1, 3).reshape(rows, cols)

    (densify(v32) @ d32).backward(dy.float())
    assert_product_close(s.data.grad, v32.grad, "dsd: gradient of the sparse values")
    assert_product_close(d.grad, d32.grad, "dsd: gradient of the dense operand")
    # sdd: gradients of both dense operands
    a = lhs.cuda().requires_grad_(True)
    b = dense_rhs.t().contiguous().cuda().requires_grad_(True)          # [inner, cols]
    out = stk.ops.sdd(a, b, topo)
    dblocks = (torch.randn(nnz, blocking, blocking, generator=g) * 0.1).half()
    out.data.backward(dblocks.cuda())
    a32 = lhs.float().requires_grad_(True)
    b32 = dense_rhs.t().contiguous().float().requires_grad_(True)
    ((a32 @ b32) * keep).backward(densify(dblocks.float()))
    assert_product_close(a.grad, a32.grad, "sdd: gradient of the left operand")
    assert_product_close(b.grad, b32.grad, "sdd: gradient of the right operand")


def test_regroup_blocks_round_trip_and_guards(stk):
    """The copy kernel alone: into zero-filled 128-blocks and back is the identity, places no block maps to
    stay zero, 1-, 2- and 4-byte elements; a slot outside the 128-blocks is skipped and reported."""
    from stk_b200.backend import kernels, lib
    from stk_b200.ops import small_blocks
    for blocking, dtype in ((16, torch.float16), (32, torch.float32), (64, torch.bfloat16), (64, torch.float8_e4m3fn)):
        topo = _topology(stk, 512, 640, 0.8, blocking, 2).to("cuda")
        coarse = small_blocks.coarse_topology(topo)
        nnz = topo.row_indices.numel()
        vals = torch.randint(1, 120, (nnz, blocking, blocking), dtype=torch.uint8).cuda()
        vals = vals.to(torch.float32).to(dtype)
        big = torch.zeros((coarse.blocks, 128, 128), dtype=dtype, device="cuda")
        kernels.regroup_blocks(vals, big, coarse.slot, True)
        back = torch.empty_like(vals)
        kernels.regroup_blocks(back, big, coarse.slot, False)
        assert torch.equal(back.view(torch.uint8), vals.view(torch.uint8))
        assert int((big.float() != 0).sum().item()) == vals.numel()        # every value is nonzero, nothing else is
        # the same matrix densified at both blockings
        fine = stk.Matrix(topo.size(), vals, topo.row_indices, topo.column_indices, topo.offsets,
                          topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
        assert torch.equal(stk.ops.to_dense(fine).view(torch.uint8),
                           stk.ops.to_dense(coarse.matrix(big)).view(torch.uint8))
    topo = _topology(stk, 256, 256, 0.5, 64, 9).to("cuda")
    coarse = small_blocks.coarse_topology(topo)
    vals = torch.rand(topo.data.shape, device="cuda").half() + 1
    big = torch.zeros((coarse.blocks, 128, 128), dtype=torch.float16, device="cuda")
    kernels.regroup_blocks(vals, big, coarse.slot, True)
    bad = coarse.slot.clone()
    bad[0] = coarse.blocks * 4
    out = torch.ones_like(vals)
    kernels.regroup_blocks(out, big, bad, False)
    assert lib.device_status() == -2           # STK_ERR_BAD_DIMS
    assert float(out[0].abs().max()) == 0.0
    assert torch.equal(out[1:], vals[1:])
    assert small_blocks.coarse_topology(topo) is coarse           # cached on the topology


def test_shapes_that_small_blocks_cannot_take(stk):
    from stk_b200.backend import kernels
    topo = _topology(stk, 192, 256, 0.5, 64, 4).to("cuda")       # 192 rows: not a multiple of 128
    with pytest.raises(kernels.DimensionError):
        stk.ops.dsd(topo, torch.zeros(256, 128, dtype=torch.float16, device="cuda"))
    topo8 = _topology(stk, 256, 256, 0.5, 8, 4).to("cuda")
    with pytest.raises(kernels.DimensionError):
        stk.ops.dsd(topo8, torch.zeros(256, 128, dtype=torch.float16, device="cuda"))


def test_small_blocks_that_fill_their_128_blocks(stk):
    """A topology whose small blocks tile their 128-blocks completely takes the copy without a zero fill."""
    rows, cols = 256, 384
    np.random.seed(6)
    keep128 = oracle.dense_mask(rows, cols, 0.5, 128).to(torch.float16)
    for blocking in (32, 64):
        g = torch.Generator().manual_seed(blocking)
        dense = keep128 * (torch.rand(rows, cols, generator=g) + 0.5).half()
        s = stk.ops.to_sparse(dense.cuda(), blocking)
        from stk_b200.ops import small_blocks
        coarse = small_blocks.coarse_topology(s)
        assert s.row_indices.numel() == coarse.blocks * (128 // blocking) ** 2
        right = (torch.randn(cols, 128, generator=g) * 0.1).half()
        assert_product_close(stk.ops.dsd(s, right.cuda()), oracle.dsd(dense, right, torch.float16), "dsd")
        left = (torch.randn(128, rows, generator=g) * 0.1).half()
        assert_product_close(stk.ops.dds(left.cuda(), s), oracle.dds(left, dense, torch.float16), "dds")
