"""GPU tests of the API surface around the products: element-wise mul (the reference's
stk/ops/eltwise_ops_test.py), autocast behaviour (stk/backend/autocast.py), externally supplied
transposed metadata in the reference's tie order, the kernel-choice statistics, the pair kernel's
work-item table, top-k routing against the host logic, and bad metadata handed to the transpose."""
import itertools

import numpy as np
import pytest
import torch

from oracle import stk_oracle as oracle
from tests.parity import assert_product_close

pytestmark = pytest.mark.gpu

_ELTWISE_SIZES = (
    (128, 128, 0.0), (256, 256, 0.5), (2048, 1024, 0.8), (512, 128, 0.0), (128, 512, 0.0),
    (1024, 512, 0.0), (1024, 512, 0.5), (1024, 512, 0.75), (512, 1024, 0.0), (512, 1024, 0.5),
    (512, 1024, 0.75), (1024, 1024, 0.0), (1024, 1024, 0.5), (1024, 1024, 0.75),
)
_DTYPE = (torch.float16, torch.bfloat16)


@pytest.fixture(scope="module")
def stk():
    import stk_b200
    from stk_b200.backend import lib
    yield stk_b200
    assert lib.device_status() == 0


def _dense_and_sparse(stk, rows, cols, sparsity, dtype, std=0.1):
    mask = stk.random.dense_mask(rows, cols, sparsity, 128)
    dense = (torch.randn(rows, cols) * std * mask).type(dtype).cuda()
    sparse = stk.ops.to_sparse(dense, 128)
    return dense.requires_grad_(True), sparse.requires_grad_(True)


@pytest.mark.parametrize("m,n,sparsity,dtype", [(*s, d) for s, d in itertools.product(_ELTWISE_SIZES, _DTYPE)])
def test_eltwise_mul(stk, m, n, sparsity, dtype):
    """stk.ops.mul forward and both gradients against torch.mul on the dense twins
    (stk/ops/eltwise_ops_test.py:53-83).  Element-wise products of 16-bit values: one rounding."""
    torch.manual_seed(m + n)
    a_dense, a = _dense_and_sparse(stk, m, n, sparsity, dtype)
    b_vals = (torch.randn_like(a.data) * 0.1).detach()
    b = stk.Matrix(a.size(), b_vals, a.row_indices, a.column_indices, a.offsets)
    b_dense = stk.ops.to_dense(b).requires_grad_(True)
    b.requires_grad_(True)
    out = stk.ops.mul(a, b)
    expected = torch.mul(a_dense, b_dense)
    expected.sum().backward()
    stk.ops.sum(out).backward()
    dense_out = stk.ops.to_dense(out)
    assert dense_out.dim() == 2 and dense_out.size() == expected.size() and dense_out.dtype == dtype
    assert torch.equal(dense_out, expected.detach())
    assert torch.equal(stk.ops.to_dense(a.grad), a_dense.grad)
    assert torch.equal(stk.ops.to_dense(b.grad), b_dense.grad)


@pytest.mark.parametrize("op", ["sdd", "dsd", "dds"])
def test_ops_under_autocast(stk, op):
    """Under torch.autocast(bfloat16) the products cast their fp32 operands to bfloat16, run with
    autocast off, and return bfloat16 (stk/backend/autocast.py:19-37); gradients flow back in fp32."""
    np.random.seed(5)
    torch.manual_seed(5)
    topo = stk.random.mask(384, 256, 0.5, 128).to("cuda")
    a32 = (torch.randn(384, 256, device="cuda") * 0.1).requires_grad_(True)
    b32 = (torch.randn(256, 256, device="cuda") * 0.1).requires_grad_(True)
    sp_vals = (torch.randn(topo.data.shape, device="cuda") * 0.1)
    bf = torch.bfloat16
    r, c = topo.row_indices.cpu().numpy(), topo.column_indices.cpu().numpy()
    with torch.autocast(device_type="cuda", dtype=bf):
        if op == "sdd":
            out = stk.ops.sdd(a32, b32, topo)
            got, ref = out.data, oracle.sdd(a32.detach().cpu().to(bf), b32.detach().cpu().to(bf), r, c, bf)
            leaves = (a32, b32)
        else:
            s = stk.Matrix(topo.size(), sp_vals.clone().requires_grad_(True), topo.row_indices,
                           topo.column_indices, topo.offsets, topo.column_indices_t, topo.offsets_t,
                           topo.block_offsets_t)
            s_dense = oracle.to_dense(sp_vals.cpu().to(bf), r, c, (384, 256))
            if op == "dsd":
                d32 = (torch.randn(256, 128, device="cuda") * 0.1).requires_grad_(True)
                got, ref = stk.ops.dsd(s, d32), oracle.dsd(s_dense, d32.detach().cpu().to(bf), bf)
            else:
                d32 = (torch.randn(128, 384, device="cuda") * 0.1).requires_grad_(True)
                got, ref = stk.ops.dds(d32, s), oracle.dds(d32.detach().cpu().to(bf), s_dense, bf)
            leaves = (s.data, d32)
        assert torch.is_autocast_enabled()
    assert got.dtype == bf
    assert_product_close(got, ref, f"{op} under autocast")
    got.float().sum().backward()
    for leaf in leaves:
        assert leaf.grad is not None and leaf.grad.dtype == torch.float32 and leaf.grad.shape == leaf.shape


@pytest.mark.parametrize("mode", ["auto", "1"])
def test_external_transposed_metadata_in_reference_tie_order(stk, golden, mode):
    """A Matrix built from all seven fields as the reference produces them: its unstable argsort leaves
    the rows inside a block column unordered (stk/matrix.py:110; fixture sq205).  The products through
    the transposed metadata must still be right - the pair kernel's merge needs ascending lists, so
    such a topology must end up on a kernel that does not."""
    from stk_b200.backend import kernels
    g = golden["metadata"]
    t = lambda k, dt: torch.from_numpy(g[f"sq205/{k}"].astype(dt)).cuda()
    cit, bot, ot = g["sq205/column_indices_t"], g["sq205/block_offsets_t"], g["sq205/offsets_t"]
    unsorted_cols = sum(1 for c in range(len(ot) - 1) if np.any(np.diff(cit[ot[c]:ot[c + 1]].astype(np.int64)) < 0))
    assert unsorted_cols > 0, "the fixture must hold the reference's non-stable order"
    nnz = len(cit)
    torch.manual_seed(2)
    data = (torch.randn(nnz, 128, 128) * 0.1).half()
    m = stk.Matrix(torch.Size((2048, 2048)), data.cuda(), t("row_indices", np.int16), t("column_indices", np.int16),
                   t("offsets", np.int32), t("column_indices_t", np.int16), t("offsets_t", np.int32),
                   t("block_offsets_t", np.int32))
    dense = oracle.to_dense(data, g["sq205/row_indices"], g["sq205/column_indices"], (2048, 2048))
    b = (torch.randn(2048, 256) * 0.1).half()
    a = (torch.randn(256, 2048) * 0.1).half()
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = mode
    try:
        for _ in range(3):          # the statistics arrive asynchronously: every call must be right
            assert_product_close(stk.ops.dsd(m.t(), b.cuda()), oracle.dsd(dense.t(), b, torch.float16), "dsd S^T")
            assert_product_close(stk.ops.dds(a.cuda(), m), oracle.dds(a, dense, torch.float16), "dds S")
            torch.cuda.synchronize()
        hints = kernels.pair_hints(m.offsets, m.row_indices, m.column_indices, 16, m.offsets_t, m.column_indices_t,
                                   need_t=True, wait=True)
        assert hints[3] is True and hints[4] is False
    finally:
        kernels.PAIR_MODE = saved


def _stats_by_hand(rows, cols):
    rp = len({(r >> 1, c) for r, c in zip(rows, cols)})
    cp = len({(r, c >> 1) for r, c in zip(rows, cols)})
    tl = len({(r >> 1, c >> 1) for r, c in zip(rows, cols)})
    return rp, cp, tl


def test_pair_stats_and_plan_match_host_logic(stk):
    from stk_b200 import dmoe
    from stk_b200.backend import kernels, lib
    L = lib.load()
    dev = torch.device("cuda", 0)
    np.random.seed(17)
    cases = [stk.random.mask(1024, 2048, 0.6, 128).to("cuda"), stk.random.mask(2048, 1024, 0.0, 128).to("cuda"),
             dmoe.block_diagonal_topology(torch.tensor([3, 0, 1, 4, 2, 5]) * 128, 512, torch.float16, "cuda")]
    for m in cases:
        rows, cols = m.row_indices.cpu().tolist(), m.column_indices.cpu().tolist()
        R, Cb = m.size()[0] // 128, m.size()[1] // 128
        stats = torch.zeros(8, dtype=torch.int32, device=dev)
        lib.check(L.stk_b200_pair_stats(lib.ptr(m.offsets), lib.ptr(m.row_indices), lib.ptr(m.column_indices),
                                        lib.ptr(m.offsets_t), lib.ptr(m.column_indices_t), R, Cb, len(rows),
                                        lib.ptr(stats), lib.stream_ptr(dev)), "stk_b200_pair_stats")
        assert stats.cpu().tolist()[:6] == [*_stats_by_hand(rows, cols), 1, 1, 1]
        # the work-item table: every list exactly once, pairs only inside runs, longest lists first
        for offsets, idx, n in ((m.offsets, m.column_indices, R), (m.offsets_t, m.column_indices_t, Cb)):
            plan = kernels.pair_plan(offsets, idx).cpu().tolist()
            off, lst = offsets.cpu().tolist(), idx.cpu().tolist()
            G, seen, costs = plan[0], [], []
            for e in plan[1:1 + G]:
                r, single = e & 0x3fffffff, (e >> 30) & 1
                seen += [r] if single else [r, r + 1]
                costs.append(off[r + 1] - off[r])
                if not single:
                    a, b = lst[off[r]:off[r + 1]], lst[off[r + 1]:off[r + 2]]
                    assert not (a and b and (a[-1] < b[0] or b[-1] < a[0])), "a pair straddles a cut"
            assert sorted(seen) == list(range(n))
            assert costs == sorted(costs, reverse=True)
    # blocks out of order are reported as such (and the counts then mean nothing)
    m = cases[0]
    perm = torch.arange(m.row_indices.numel() - 1, -1, -1, device=dev)
    stats = torch.zeros(8, dtype=torch.int32, device=dev)
    ri, ci = m.row_indices[perm].contiguous(), m.column_indices[perm].contiguous()
    lib.check(L.stk_b200_pair_stats(lib.ptr(m.offsets), lib.ptr(ri), lib.ptr(ci), None, None, 8, 16, ri.numel(),
                                    lib.ptr(stats), lib.stream_ptr(dev)), "stk_b200_pair_stats")
    assert stats.cpu().tolist()[3:6] == [0, -1, 1]


def test_topk_routing_kernels_match_host_logic(stk):
    from stk_b200 import dmoe
    from tests.test_dmoe_host import check_topk
    g = torch.Generator().manual_seed(4)
    for tokens, experts, k, hidden in [(3000, 8, 2, 64), (16384, 64, 2, 128), (500, 5, 3, 8)]:
        ids = torch.randint(0, experts, (tokens, k), generator=g)
        if experts == 64:
            ids[ids == 9] = 10         # an expert without tokens
        x = torch.randn(tokens, hidden, generator=g)
        w = torch.rand(tokens, k, generator=g)
        check_topk(dmoe, x.half().cuda(), ids.cuda().to(torch.int32), w.cuda(), experts, tol=4e-3)
        dev_res = dmoe.route_topk(ids.cuda().to(torch.int32), experts)
        host_res = dmoe.route_topk(ids, experts)
        for a, b in zip(dev_res, host_res):
            if torch.is_tensor(a):
                assert torch.equal(a.cpu(), b.cpu())
            else:
                assert a == b
        # 16-bit rows: the device kernel (fp32 accumulate, one rounding) against the host formula
        xh = x.half()
        index, position = dev_res[0], dev_res[1]
        yp = dmoe.permute_tokens(xh.cuda(), index, dev_res[4], top_k=k)
        got = dmoe.combine_tokens(yp, position, w.cuda(), tokens, k)
        expect = (xh.float() * w.sum(1, keepdim=True))
        assert torch.allclose(got.float().cpu(), expect, rtol=2e-3, atol=2e-3)


def test_transpose_skips_and_reports_bad_column_indices(stk):
    """A column index outside [0, block_cols) never reaches the counters: the block is left out (as
    the reference's histc drops out-of-range values) and STK_ERR_BAD_DIMS is recorded."""
    from stk_b200.backend import kernels, lib
    for nnz, block_cols in ((64, 8), (40000, 2048)):       # single-CTA path and multi-kernel path
        rows = torch.arange(nnz, dtype=torch.int16, device="cuda") % 7
        cols = (torch.arange(nnz, device="cuda") % block_cols).to(torch.int16)
        cols[nnz // 2] = block_cols + 5
        cols[nnz // 3] = -3
        cit, ot, bot = kernels.transpose_meta(rows, cols, block_cols)
        torch.cuda.synchronize()
        assert lib.device_status() == -2
        good = (cols >= 0) & (cols < block_cols)
        counts = torch.bincount(cols[good].long(), minlength=block_cols)
        assert torch.equal(ot.cpu()[1:].long(), torch.cumsum(counts, 0).cpu())
        assert int(ot[-1]) == nnz - 2


def test_topology_kernel_refuses_bins_that_do_not_add_up(stk):
    """The dMoE topology kernel sizes nothing itself: bins that are negative or whose sum is not the
    number of block rows the arrays were allocated for must leave the arrays untouched and record
    STK_ERR_BAD_DIMS (they used to be trusted, and positions computed from them were written)."""
    from stk_b200 import dmoe
    from stk_b200.backend import lib
    good = dmoe.topology_from_bins(torch.tensor([2, 0, 3], dtype=torch.int32, device="cuda"), 5, 256,
                                   torch.float16, "cuda")
    torch.cuda.synchronize()
    assert lib.device_status() == 0
    assert good.offsets_t.tolist() == [0, 2, 4, 4, 4, 7, 10]
    for bins, block_rows in (([4096, 4096], 64), ([2, -1, 4], 5), ([1, 1, 1], 5)):
        dmoe.topology_from_bins(torch.tensor(bins, dtype=torch.int32, device="cuda"), block_rows, 256,
                                torch.float16, "cuda")
        torch.cuda.synchronize()
        assert lib.device_status() == -2


def test_gather_blocks_never_reads_a_block_outside_the_matrix(stk):
    """A block index outside [0, block rows) x [0, block columns) used to be turned into an address; it
    now yields a block of zeros and STK_ERR_BAD_DIMS, in the 16-byte kernel and in the element-wise one."""
    from stk_b200.backend import kernels, lib
    for blocking, dtype in ((128, torch.float16), (4, torch.float32)):
        x = torch.randn(4 * blocking, 3 * blocking, device="cuda").to(dtype)
        rows = torch.tensor([0, 3, 7, 1], dtype=torch.int16, device="cuda")       # 7: outside
        cols = torch.tensor([2, 0, 1, -1], dtype=torch.int16, device="cuda")      # -1: outside
        data = kernels.gather_blocks(x, blocking, rows, cols)
        torch.cuda.synchronize()
        assert lib.device_status() == -2
        b = blocking
        assert torch.equal(data[0], x[0:b, 2 * b:3 * b]) and torch.equal(data[1], x[3 * b:4 * b, 0:b])
        assert not data[2].any() and not data[3].any()


def _as_int32(stk, m):
    i32 = lambda t: t.to(torch.int32)
    return stk.Matrix(m.size(), m.data, i32(m.row_indices), i32(m.column_indices), m.offsets)


@pytest.mark.parametrize("mode", ["0", "1", "2", "3", "auto"])
def test_int32_block_indices_give_identical_results(stk, mode):
    """The same topology with int32 instead of int16 block indices: transposed metadata equal value for
    value, every product bit-identical, conversions bit-identical (the reference leaves the index
    dtype as a TODO, stk/matrix.py:178-181)."""
    from stk_b200 import dmoe
    from stk_b200.backend import kernels
    np.random.seed(23)
    torch.manual_seed(23)
    cases = [stk.random.randn((512, 768), 0.5, 128).to("cuda"),
             dmoe.block_diagonal_topology(torch.tensor([2, 1, 0, 3]) * 128, 256, torch.float16, "cuda")]
    cases[1].data.normal_(0, 0.1)
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = mode
    try:
        for m16 in cases:
            m32 = _as_int32(stk, m16)
            m32.validate()
            assert m32.column_indices_t.dtype == torch.int32 and m32.row_indices.dtype == torch.int32
            assert torch.equal(m32.column_indices_t.to(torch.int16), m16.column_indices_t)
            assert torch.equal(m32.offsets_t, m16.offsets_t) and torch.equal(m32.block_offsets_t, m16.block_offsets_t)
            rows, cols = m16.size()
            a = (torch.randn(rows, 256, device="cuda") * 0.1).half()
            b = (torch.randn(256, cols, device="cuda") * 0.1).half()
            right = (torch.randn(cols, 256, device="cuda") * 0.1).half()
            left = (torch.randn(256, rows, device="cuda") * 0.1).half()
            for _ in range(2):         # the second round runs with the kernel-choice statistics known
                assert torch.equal(stk.ops.sdd(a, b, m32).data, stk.ops.sdd(a, b, m16).data)
                assert torch.equal(stk.ops.dsd(m32, right), stk.ops.dsd(m16, right))
                assert torch.equal(stk.ops.dsd(m32.t(), left.t()), stk.ops.dsd(m16.t(), left.t()))
                assert torch.equal(stk.ops.dds(left, m32), stk.ops.dds(left, m16))
                assert torch.equal(stk.ops.dds(right.t(), m32.t()), stk.ops.dds(right.t(), m16.t()))
                torch.cuda.synchronize()
            assert torch.equal(stk.ops.to_dense(m32), stk.ops.to_dense(m16))
            ri = stk.ops.row_indices(m32.size(), m32.data, m32.offsets, m32.column_indices)
            assert ri.dtype == torch.int32 and torch.equal(ri, m32.row_indices)
            again = stk.ops.to_sparse(stk.ops.to_dense(m16), 128, index_dtype=torch.int32)
            assert again.column_indices.dtype == torch.int32
            keep = (m16.data.view(m16.data.shape[0], -1) != 0).any(1)
            assert torch.equal(again.data, m16.data[keep])
    finally:
        kernels.PAIR_MODE = saved


def test_more_than_32767_blocks_per_side(stk):
    """40000 block rows (blocking 1): beyond what int16 indices can name.  The reference raises
    (stk/matrix.py:161-167); here the conversion switches to int32 indices and round-trips exactly."""
    torch.manual_seed(3)
    x = torch.randn(40000, 16).half() * (torch.rand(40000, 16) < 0.3)
    m = stk.ops.to_sparse(x.cuda(), 1)
    m.validate()
    assert m.row_indices.dtype == torch.int32 and m.column_indices.dtype == torch.int32
    nz = torch.nonzero(x != 0)
    assert torch.equal(m.row_indices.cpu().long(), nz[:, 0]) and torch.equal(m.column_indices.cpu().long(), nz[:, 1])
    assert torch.equal(stk.ops.to_dense(m).cpu(), x)
    order = torch.argsort(nz[:, 1], stable=True)
    assert torch.equal(m.block_offsets_t.cpu().long(), order)
    assert torch.equal(m.column_indices_t.cpu().long(), nz[:, 0][order])
    # blocks of 8 x 8 on a matrix with 40000 block rows: the strip kernels take several launches
    y = (torch.randn(40000 * 8, 16) * (torch.rand(40000, 1, 2, 1) < 0.5).expand(40000, 8, 2, 8).reshape(320000, 16)).half()
    m8 = stk.ops.to_sparse(y.cuda(), 8)
    assert m8.row_indices.dtype == torch.int32
    assert torch.equal(stk.ops.to_dense(m8).cpu(), y)
    with pytest.raises(ValueError):
        stk.Matrix(m.size(), m.data, m.row_indices.to(torch.int16), m.column_indices.to(torch.int16), m.offsets,
                   m.column_indices_t, m.offsets_t, m.block_offsets_t)



@pytest.mark.parametrize("mode", ["0", "1", "2", "auto"])
def test_float8_products_match_the_dequantized_reference(stk, mode):
    """float8_e4m3fn operands (an extension): every product, in every operand layout the 16-bit products
    take (row- / column-major dense operands, blocks as stored or transposed), equals the fp32 product of
    the dequantized operands up to the one bfloat16 rounding of the result - in the 128x128 kernel and on
    CTA pairs in both shapes, for a K that is not a multiple of a pipeline stage (416 = 3 * 128 + 32)."""
    from stk_b200 import dmoe
    from stk_b200.backend import kernels
    F8 = torch.float8_e4m3fn
    np.random.seed(31)
    torch.manual_seed(31)
    cases = [stk.random.randn((512, 768), 0.5, 128).to("cuda"),
             dmoe.block_diagonal_topology(torch.tensor([2, 1, 0, 3]) * 128, 256, torch.float16, "cuda")]
    cases[1].data.normal_(0, 0.5)
    rand8 = lambda *shape: torch.randn(*shape, device="cuda").to(F8)
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = mode
    try:
        for topo in cases:
            rows, cols = topo.size()
            dense16 = lambda m: stk.ops.to_dense(m).float()
            pattern = dense16(stk.ops.ones_like(topo))
            s8 = stk.Matrix(topo.size(), (topo.data.float() * 2).to(F8), topo.row_indices, topo.column_indices,
                            topo.offsets, topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
            s8.validate()
            s_dense = dense16(stk.Matrix(topo.size(), s8.data.to(torch.bfloat16), topo.row_indices,
                                         topo.column_indices, topo.offsets, topo.column_indices_t,
                                         topo.offsets_t, topo.block_offsets_t))
            for _ in range(2):          # the second round runs with the kernel-choice statistics known
                # sdd: [rows, 416] x [416, cols] on the topology, the four layout combinations
                a, at = rand8(rows, 416), rand8(416, rows)            # lhs row-major / stored transposed
                b, bt = rand8(416, cols), rand8(cols, 416)            # rhs row-major / stored transposed
                for lhs in (a, at.t()):
                    for rhs in (b, bt.t()):
                        ref = (lhs.float() @ rhs.float()) * pattern
                        out = stk.ops.sdd(lhs, rhs, topo)
                        assert out.data.dtype == torch.bfloat16
                        assert_product_close(dense16(out), ref, "fp8 sdd")
                gelu = stk.ops.sdd_gelu(a, bt.t(), topo)
                ref = (a.float() @ bt.float().t()) * pattern
                assert_product_close(dense16(gelu), torch.nn.functional.gelu(ref) * pattern, "fp8 sdd + gelu")
                # dsd: op(S) x dense, S as stored and transposed, dense row- and column-major
                for op_s, op_dense, inner in ((s8, s_dense, cols), (s8.t(), s_dense.t(), rows)):
                    r, rt = rand8(inner, 256), rand8(256, inner)
                    for rhs in (r, rt.t()):
                        y = stk.ops.dsd(op_s, rhs)
                        assert y.dtype == torch.bfloat16
                        assert_product_close(y, op_dense @ rhs.float(), "fp8 dsd")
                # dds: dense x op(S)
                for op_s, op_dense, inner in ((s8, s_dense, rows), (s8.t(), s_dense.t(), cols)):
                    l, lt = rand8(256, inner), rand8(inner, 256)
                    for lhs in (l, lt.t()):
                        assert_product_close(stk.ops.dds(lhs, op_s), lhs.float() @ op_dense, "fp8 dds")
    finally:
        kernels.PAIR_MODE = saved


def test_float8_matrices_convert_like_16_bit_ones(stk):
    """to_sparse / to_dense / ones_like of float8_e4m3fn data (element-wise kernels): the same topology and
    the same values as the bfloat16 matrix they were quantised from, -0 counting as zero."""
    F8 = torch.float8_e4m3fn
    torch.manual_seed(5)
    for blocking in (128, 16):
        keep = (torch.rand(6, 5) < 0.4).repeat_interleave(blocking, 0).repeat_interleave(blocking, 1)
        dense = (torch.randn(6 * blocking, 5 * blocking) * keep).to(F8)
        dense[:blocking, :blocking] = torch.tensor(-0.0).to(F8)           # a block of -0: not a block
        wide = dense.to(torch.bfloat16).cuda()
        m8, m16 = stk.ops.to_sparse(dense.cuda(), blocking), stk.ops.to_sparse(wide, blocking)
        m8.validate()
        assert m8.data.dtype == F8
        for a, b in ((m8.row_indices, m16.row_indices), (m8.column_indices, m16.column_indices), (m8.offsets, m16.offsets),
                     (m8.column_indices_t, m16.column_indices_t), (m8.block_offsets_t, m16.block_offsets_t)):
            assert torch.equal(a, b)
        assert torch.equal(m8.data.view(torch.uint8), m16.data.to(F8).view(torch.uint8))
        back = stk.ops.to_dense(m8)
        assert back.dtype == F8 and torch.equal(back.to(torch.bfloat16), stk.ops.to_dense(m16))


@pytest.mark.parametrize("mode", ["1", "2"])
def test_tiny_products_launched_back_to_back_stay_exact(stk, mode):
    """Thousands of launches on topologies whose work items are one to three blocks long, different kinds of
    products following one another without a pause: every result is bit-identical to the first, and no
    bounded wait runs out.  (The end-of-stream tag of the CTA-pair kernels once raced with the MMA
    issuer's probe of the next stage; a launch in a few thousand then hung until its wait limit.)"""
    from stk_b200 import dmoe
    from stk_b200.backend import kernels, lib
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = mode
    try:
        for experts, cols_per_expert in ((5, 3), (80, 1)):
            g = torch.Generator().manual_seed(experts)
            bin_rows = torch.randint(1, 4, (experts,), generator=g)
            bin_rows[experts // 2] = 0
            topo = dmoe.block_diagonal_topology(bin_rows * 128, cols_per_expert * 128, torch.float16, "cuda")
            rows, cols = topo.size()
            a = (torch.randn(rows, 256, generator=g) * 0.1).half().cuda()
            b = (torch.randn(256, cols, generator=g) * 0.1).half().cuda()
            right = (torch.randn(cols, 384, generator=g) * 0.1).half().cuda()
            left_t = (torch.randn(rows, 384, generator=g) * 0.1).half().cuda()
            got = stk.ops.sdd(a, b, topo)
            products = {"dsd": lambda: stk.ops.dsd(got, right), "dsd T": lambda: stk.ops.dsd(got.t(), left_t),
                        "dds": lambda: stk.ops.dds(left_t.t(), got), "sdd": lambda: stk.ops.sdd(a, b, topo).data}
            for name, fn in products.items():
                first = fn().clone()
                different = 0
                for i in range(500):
                    out = fn()
                    if i % 3 == 0:
                        stk.ops.sdd(a, b, topo)
                    if i % 5 == 0:
                        stk.ops.dsd(got, right)
                    different += int(not torch.equal(out, first))
                torch.cuda.synchronize()
                assert different == 0, f"{name}: {different} of 500 results differ from the first"
                assert lib.device_status() == 0, name
    finally:
        kernels.PAIR_MODE = saved


def test_first_product_of_a_fresh_autograd_thread():
    """The backward pass runs on a worker thread that has no CUDA context bound until some runtime call binds
    one; when its first work is a product whose buffers come out of the allocator's cache, the tensor-map
    encoding is that thread's first driver call (it once answered CUDA_ERROR_INVALID_CONTEXT).  A fresh
    process, so that the worker thread is new."""
    import subprocess
    import sys
    script = r"""
import numpy as np, torch
import stk_b200 as stk
from stk_b200.backend import kernels, lib
kernels.PAIR_MODE = "0"
np.random.seed(1)
topo = stk.random.mask(256, 384, 0.0, 128).to("cuda")
vals = (torch.randn(6, 128, 128) * 0.1).half().cuda().requires_grad_(True)
s = stk.Matrix(topo.size(), vals, topo.row_indices, topo.column_indices, topo.offsets,
               topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
d = (torch.randn(384, 128) * 0.1).half().cuda()
warm = torch.empty(6, 128, 128, dtype=torch.float16, device="cuda")   # the backward's buffer will reuse this
del warm
out = stk.ops.dsd(s, d)
out.backward(torch.ones_like(out))
want = torch.ones(256, 128).double() @ d.double().cpu().t()
got = stk.ops.to_dense(stk.Matrix(topo.size(), vals.grad, topo.row_indices, topo.column_indices, topo.offsets,
                                  topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)).double().cpu()
assert (got - want).abs().max().item() < 0.05, (got - want).abs().max().item()
assert lib.device_status() == 0
print("fresh thread ok")
"""
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    done = subprocess.run([sys.executable, "-c", script], cwd=root, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "fresh thread ok" in done.stdout, done.stdout[-2000:] + done.stderr[-2000:]
