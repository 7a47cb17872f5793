"""GPU parity tests: the CUDA path (through the C ABI) against the oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

from oracle import stk_oracle as oracle
from tests import cases
from tests.parity import assert_product_close, bits

pytestmark = pytest.mark.gpu

META_KEYS = ("row_indices", "column_indices", "offsets", "column_indices_t", "offsets_t",
             "block_offsets_t")


@pytest.fixture(scope="module", params=["0", "1", "2", "3", "auto"], ids=["tile128", "pair256", "wide512", "row256", "auto"])
def stk(request):
    """The package with the matmul kernel choice forced (128x128 tiles per CTA / 256x256 supertiles
    on CTA pairs) or left to the per-topology heuristic."""
    import stk_b200
    from stk_b200.backend import kernels, lib
    assert torch.cuda.is_available()
    lib.load()
    saved = kernels.PAIR_MODE
    kernels.PAIR_MODE = request.param
    yield stk_b200
    kernels.PAIR_MODE = saved
    assert lib.device_status() == 0, "a kernel reported a bounded wait that ran out"


def _check_meta(m, expect, what):
    for key in META_KEYS:
        mine = getattr(m, key).cpu().numpy()
        assert mine.dtype == expect[key].dtype, f"{what}: dtype of {key}"
        np.testing.assert_array_equal(mine, expect[key], err_msg=f"{what}: {key}")


@pytest.mark.parametrize("name", sorted(cases.METADATA_CASES))
def test_random_mask_bit_exact(stk, golden, name):
    g = golden["metadata"]
    rows, cols, sparsity, blocking, seed = cases.METADATA_CASES[name]
    np.random.seed(seed)
    m = stk.random.mask(rows, cols, sparsity, blocking)
    m.validate()
    assert tuple(m.data.shape) == tuple(g[f"{name}/data_shape"])
    assert m.data.dtype == torch.float16 and bool((m.data == 1).all())
    # oracle (stable tie order) ...
    np.random.seed(seed)
    _check_meta(m, oracle.mask(rows, cols, sparsity, blocking), name)
    # ... and the reference's own output, tie order canonicalised
    for key in ("row_indices", "column_indices", "offsets", "offsets_t"):
        np.testing.assert_array_equal(getattr(m, key).numpy(), g[f"{name}/{key}"])
    cit, bot = oracle.canonical_tie_order(g[f"{name}/column_indices_t"], g[f"{name}/offsets_t"],
                                          g[f"{name}/block_offsets_t"])
    np.testing.assert_array_equal(m.column_indices_t.numpy(), cit)
    np.testing.assert_array_equal(m.block_offsets_t.numpy(), bot)


@pytest.mark.parametrize("name", sorted(cases.CONVERT_CASES))
def test_conversion_bit_exact(stk, golden, name):
    g = golden["convert"]
    rows, cols, sparsity, blocking, seed, dtype = cases.CONVERT_CASES[name]
    x = cases.convert_input(name)
    m = stk.ops.to_sparse(x.cuda(), blocking)
    assert m.is_cuda and m.size() == x.size()
    _check_meta(m, oracle.to_sparse(x, blocking), name)
    assert tuple(m.data.shape) == tuple(g[f"{name}/data_shape"])
    np.testing.assert_array_equal(bits(m.data).ravel(), g[f"{name}/data_bits"].ravel())
    dense = stk.ops.to_dense(m)
    np.testing.assert_array_equal(bits(dense), g[f"{name}/dense_bits"].reshape(rows, cols))
    ri = stk.ops.row_indices(m.size(), m.data, m.offsets, m.column_indices)
    assert ri.dtype == torch.int16
    np.testing.assert_array_equal(ri.cpu().numpy(), g[f"{name}/row_indices"])
    # host tensors are staged through the GPU and come back to the host
    mh = stk.ops.to_sparse(x, blocking)
    assert not mh.is_cuda
    np.testing.assert_array_equal(bits(mh.data).ravel(), g[f"{name}/data_bits"].ravel())
    np.testing.assert_array_equal(bits(stk.ops.to_dense(mh)), bits(dense))


# The reference's conversion test, stk/ops/matrix_ops_test.py:26-58.
@pytest.mark.parametrize("rows,cols,sparsity,blocking", [
    (8, 16, 0.0, 1), (8, 16, 0.5, 1), (8, 16, .95, 1), (16, 8, 0.0, 1), (16, 8, 0.5, 1),
    (16, 8, .95, 1), (8, 16, 0.0, 8), (8, 16, 0.5, 8), (8, 16, 1.0, 8), (16, 8, 0.0, 8),
    (16, 8, 0.5, 8), (16, 8, 1.0, 8), (128, 256, 0.5, 16), (256, 128, 0.75, 32),
    (512, 512, .875, 128)])
def test_format_conversion_round_trip(stk, rows, cols, sparsity, blocking):
    mask = stk.random.dense_mask(rows, cols, sparsity, blocking)
    assert mask.shape == (rows, cols)
    assert set(mask.unique().tolist()) <= {0.0, 1.0}
    x = (torch.randn(rows, cols) * mask).type(torch.float16)
    sparse_x = stk.ops.to_sparse(x, blocking)
    sparse_x.validate()
    assert sparse_x.dim() == 2 and tuple(sparse_x.size()) == (rows, cols)
    numblocks = rows // blocking * cols // blocking
    nnz = round(numblocks * (1 - sparsity)) * blocking ** 2
    assert sparse_x.nnz == nnz
    dense_x = stk.ops.to_dense(sparse_x)
    assert tuple(dense_x.shape) == (rows, cols)
    assert torch.count_nonzero(dense_x).item() == nnz
    assert torch.all(torch.eq(x, dense_x))
    # stk/random/random_ops_test.py:49-69
    m = stk.random.mask(rows, cols, sparsity, blocking)
    m.validate()
    assert m.nnz == nnz and bool((m.data == 1).all())


@pytest.mark.parametrize("shape", [(64, 2048, 0.3), (300, 300, 0.6), (2112, 7168, 0.016),
                                   (16, 32767, 0.01), (1, 1, 1.0), (40, 1536, 0.5)])
def test_transpose_meta_bit_exact(stk, shape):
    """Both transpose paths (single-CTA and multi-kernel) against the stable-sort oracle."""
    from stk_b200.backend import kernels
    block_rows, block_cols, density = shape
    rng = np.random.default_rng(block_rows * 7 + block_cols)
    r, c = np.nonzero(rng.random((block_rows, block_cols)) < density)
    r16, c16 = r.astype(np.int16), c.astype(np.int16)
    expect = oracle.transpose(block_cols, r16, c16)
    got = kernels.transpose_meta(torch.from_numpy(r16).cuda(), torch.from_numpy(c16).cuda(),
                                 block_cols)
    for a, b in zip(got, expect):
        assert a.cpu().numpy().dtype == b.dtype
        np.testing.assert_array_equal(a.cpu().numpy(), b)
    cit, offt, bot = (t.cpu().numpy() for t in got)
    # invariants that hold for any valid transpose
    assert np.array_equal(np.sort(bot), np.arange(len(r)))
    assert np.all(np.diff(c16[bot].astype(np.int64)) >= 0)
    assert np.array_equal(r16[bot], cit)


def _gpu_product(stk, name):
    op, trans_a, trans_b, dtype = cases.MATMUL_CASES[name]
    inp = cases.matmul_inputs(name)
    dev = "cuda"
    meta = [torch.from_numpy(inp[k]).to(dev) for k in ("row_indices", "column_indices", "offsets")]
    if op == "sdd":
        topo = stk.Matrix(inp["topo_shape"], torch.empty(len(inp["row_indices"]), 128, 128,
                                                        dtype=dtype, device=dev), *meta)
        a, b = inp["a"].to(dev), inp["b"].to(dev)
        return stk.ops.sdd(a.t() if trans_a else a, b.t() if trans_b else b, topo).data
    s = stk.Matrix(inp["sparse_shape"], inp["data"].to(dev), *meta)
    d = inp["dense"].to(dev)
    if op == "dsd":
        return stk.ops.dsd(s.t() if trans_a else s, d.t() if trans_b else d)
    return stk.ops.dds(d.t() if trans_a else d, s.t() if trans_b else s)


@pytest.mark.parametrize("name", sorted(cases.MATMUL_CASES))
def test_products_match_reference_kernels(stk, golden, name):
    """Against the outputs of the reference's own kernels and against the oracle."""
    from tests.test_oracle import _from_bits, oracle_product
    g = golden["matmul"]
    dtype = cases.MATMUL_CASES[name][3]
    out = _gpu_product(stk, name)
    assert out.dtype == dtype and out.is_contiguous()
    ref = _from_bits(g[f"{name}/out_bits"], g[f"{name}/out_shape"], dtype)
    assert_product_close(out, ref, name + " vs reference kernels")
    assert_product_close(out, oracle_product(name), name + " vs oracle")


def test_c1_all_ops(stk):
    """The benchmark's CPU-runnable configuration: seed-0 1024x1024 topology at 25 % density,
    A [1024,512], B [512,1024] ~ N(0, 0.02), fp16; every op and transpose against the oracle."""
    np.random.seed(0)
    torch.manual_seed(0)
    topo = stk.random.mask(1024, 1024, 0.75, 128)
    np.testing.assert_array_equal(topo.block_offsets_t.numpy(),
                                  [0, 7, 3, 12, 13, 1, 4, 15, 8, 10, 5, 14, 2, 6, 9, 11])
    a = (torch.randn(1024, 512) * 0.02).half()
    b = (torch.randn(512, 1024) * 0.02).half()
    r, c = topo.row_indices.numpy(), topo.column_indices.numpy()
    topo_d = topo.to("cuda")
    for ta in (False, True):
        for tb in (False, True):
            A = a.t().contiguous().cuda().t() if ta else a.cuda()
            B = b.t().contiguous().cuda().t() if tb else b.cuda()
            out = stk.ops.sdd(A, B, topo_d)
            assert_product_close(out.data, oracle.sdd(a, b, r, c, torch.float16), f"sdd {ta}{tb}")
    vals = (torch.randn(16, 128, 128) * 0.02).half()
    s = stk.Matrix(topo.size(), vals.cuda(), topo_d.row_indices, topo_d.column_indices,
                   topo_d.offsets, topo_d.column_indices_t, topo_d.offsets_t,
                   topo_d.block_offsets_t)
    s_dense = oracle.to_dense(vals, r, c, (1024, 1024))
    d = (torch.randn(1024, 512) * 0.02).half()
    for ts in (False, True):
        for td in (False, True):
            D = d.t().contiguous().cuda().t() if td else d.cuda()
            S = s.t() if ts else s
            SD = s_dense.t() if ts else s_dense
            assert_product_close(stk.ops.dsd(S, D), oracle.dsd(SD, d, torch.float16), f"dsd {ts}{td}")
            Dt = d.t().cuda() if not td else d.cuda().t()  # [512, 1024] logical either way
            Dt_ref = d.t()
            assert_product_close(stk.ops.dds(Dt, S), oracle.dds(Dt_ref, SD, torch.float16),
                                 f"dds {td}{ts}")


def test_empty_and_ragged(stk):
    dev = "cuda"
    # no blocks at all: SDD is a no-op, DSD / DDS give zeros
    x = torch.zeros(256, 384, dtype=torch.float16, device=dev)
    e = stk.ops.to_sparse(x, 128)
    assert e.data.shape == (0, 128, 128) and e.offsets.tolist() == [0, 0, 0]
    assert e.offsets_t.tolist() == [0, 0, 0, 0]
    a = torch.randn(256, 64, dtype=torch.float16, device=dev)
    b = torch.randn(64, 384, dtype=torch.float16, device=dev)
    assert stk.ops.sdd(a, b, e).data.shape == (0, 128, 128)
    d = torch.randn(384, 128, dtype=torch.float16, device=dev)
    assert torch.count_nonzero(stk.ops.dsd(e, d)).item() == 0
    d2 = torch.randn(128, 256, dtype=torch.float16, device=dev)
    out = stk.ops.dds(d2, e)
    assert out.shape == (128, 384) and torch.count_nonzero(out).item() == 0
    # empty block rows and columns inside a non-empty matrix
    y = torch.zeros(512, 512, dtype=torch.bfloat16)
    y[128:256, 256:384] = torch.randn(128, 128).bfloat16()
    y[384:, :128] = torch.randn(128, 128).bfloat16()
    s = stk.ops.to_sparse(y.cuda(), 128)
    assert s.offsets.tolist() == [0, 0, 1, 1, 2] and s.offsets_t.tolist() == [0, 1, 1, 2, 2]
    d = (torch.randn(512, 256) * 0.1).bfloat16()
    assert_product_close(stk.ops.dsd(s, d.cuda()), oracle.dsd(y, d, torch.bfloat16), "ragged dsd")
    assert_product_close(stk.ops.dsd(s.t(), d.cuda()), oracle.dsd(y.t(), d, torch.bfloat16), "ragged dsd t")
    d = (torch.randn(256, 512) * 0.1).bfloat16()
    assert_product_close(stk.ops.dds(d.cuda(), s), oracle.dds(d, y, torch.bfloat16), "ragged dds")
    assert_product_close(stk.ops.dds(d.cuda(), s.t()), oracle.dds(d, y.t(), torch.bfloat16), "ragged dds t")


def test_sdd_inner_dimension_not_multiple_of_64(stk):
    """K only has to be a multiple of 32 (stk/backend/triton_kernels.py:15-19)."""
    np.random.seed(3)
    topo = stk.random.mask(256, 384, 0.5, 128).to("cuda")
    for k in (32, 96, 224):
        a = (torch.randn(256, k) * 0.1).half()
        b = (torch.randn(k, 384) * 0.1).half()
        ref = oracle.sdd(a, b, topo.row_indices.cpu().numpy(), topo.column_indices.cpu().numpy(),
                         torch.float16)
        assert_product_close(stk.ops.sdd(a.cuda(), b.cuda(), topo).data, ref, f"K={k}")
        assert_product_close(stk.ops.sdd(a.t().contiguous().cuda().t(),
                                         b.t().contiguous().cuda().t(), topo).data, ref, f"K={k} TT")


def test_strided_views_and_errors(stk):
    np.random.seed(5)
    topo = stk.random.mask(256, 256, 0.5, 128).to("cuda")
    big = (torch.randn(256, 512, device="cuda") * 0.1).half()
    a = big[:, 128:256 + 128]            # row-major view with a leading dimension of 512
    b = (torch.randn(256, 256, device="cuda") * 0.1).half()[::1, :]
    ref = oracle.sdd(a.cpu(), b.cpu(), topo.row_indices.cpu().numpy(),
                     topo.column_indices.cpu().numpy(), torch.float16)
    assert_product_close(stk.ops.sdd(a, b, topo).data, ref, "ld view")
    odd = big[:, 1:257]                  # misaligned view: made contiguous by the launcher
    ref = oracle.sdd(odd.cpu(), b.cpu(), topo.row_indices.cpu().numpy(),
                     topo.column_indices.cpu().numpy(), torch.float16)
    assert_product_close(stk.ops.sdd(odd, b, topo).data, ref, "misaligned view")
    with pytest.raises((AssertionError, ValueError)):
        stk.ops.sdd(a[:, :100], b[:100], topo)      # K not a multiple of 32
    with pytest.raises((AssertionError, ValueError)):
        stk.ops.dsd(topo, b[:128])                  # inner dimensions differ
    with pytest.raises(ValueError):
        stk.ops.sdd(a.float(), b.float(), topo)     # unsupported dtype
    with pytest.raises(RuntimeError):
        stk.ops.sdd(a.cpu(), b.cpu(), topo)         # no CPU path


@pytest.mark.parametrize("experts,cols_per_expert", [(5, 3), (9, 2), (80, 1)])
def test_block_diagonal_topologies_with_odd_runs(stk, experts, cols_per_expert):
    """Expert bins of 1 to 3 block rows: runs of odd length (a single row closes them), runs of one
    row, and - with 80 experts - a long work-item table.  All six products against the dense path."""
    from stk_b200 import dmoe
    g = torch.Generator().manual_seed(experts)
    bin_rows = torch.randint(1, 4, (experts,), generator=g)
    bin_rows[experts // 2] = 0                              # an expert without tokens
    f = cols_per_expert * 128
    topo = dmoe.block_diagonal_topology(bin_rows * 128, f, torch.float16, "cuda")
    rows, cols = topo.size()
    ri, ci = topo.row_indices.cpu().numpy(), topo.column_indices.cpu().numpy()
    a = (torch.randn(rows, 256, generator=g) * 0.1).half()
    b = (torch.randn(256, cols, generator=g) * 0.1).half()
    got = stk.ops.sdd(a.cuda(), b.cuda(), topo)
    assert_product_close(got.data, oracle.sdd(a, b, ri, ci, torch.float16), "sdd")
    assert_product_close(stk.ops.sdd(a.t().contiguous().cuda().t(), b.t().contiguous().cuda().t(), topo).data,
                         oracle.sdd(a, b, ri, ci, torch.float16), "sdd TT")
    s_dense = oracle.to_dense(got.data.cpu(), ri, ci, (rows, cols))
    right = (torch.randn(cols, 384, generator=g) * 0.1).half()
    left = (torch.randn(384, rows, generator=g) * 0.1).half()
    assert_product_close(stk.ops.dsd(got, right.cuda()), oracle.dsd(s_dense, right, torch.float16), "dsd")
    assert_product_close(stk.ops.dsd(got.t(), left.t().contiguous().cuda()),
                         oracle.dsd(s_dense.t(), left.t(), torch.float16), "dsd T")
    assert_product_close(stk.ops.dds(left.cuda(), got), oracle.dds(left, s_dense, torch.float16), "dds")
    assert_product_close(stk.ops.dds(right.t().contiguous().cuda(), got.t()),
                         oracle.dds(right.t(), s_dense.t(), torch.float16), "dds T")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_expert_mlp_matches_unfused_autograd(stk, dtype):
    """dmoe.expert_mlp (GeLU and its backward inside the products' epilogues) against
    sdd -> torch gelu -> dsd differentiated by autograd, forward and all three gradients."""
    from stk_b200 import dmoe
    g = torch.Generator().manual_seed(21)
    bin_rows = torch.tensor([3, 1, 0, 2, 4])
    h, f = 256, 384
    topo = dmoe.block_diagonal_topology(bin_rows * 128, f, dtype, "cuda")
    rows, cols = topo.size()
    mk = lambda *shape, scale: (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()
    x, w1, w2, dy = mk(rows, h, scale=1.0), mk(h, cols, scale=0.08), mk(cols, h, scale=0.08), mk(rows, h, scale=1.0)
    leaves = [t.clone().requires_grad_(True) for t in (x, w1, w2)]
    y = dmoe.expert_mlp(leaves[0], leaves[1], leaves[2], topo)
    y.backward(dy)
    ref_leaves = [t.clone().float().requires_grad_(True) for t in (x, w1, w2)]
    mask = oracle.to_dense(torch.ones(topo.data.shape), topo.row_indices.cpu().numpy(),
                           topo.column_indices.cpu().numpy(), (rows, cols)).cuda()
    pre = (ref_leaves[0] @ ref_leaves[1]) * mask
    y_ref = (torch.nn.functional.gelu(pre) * mask) @ ref_leaves[2]
    y_ref.backward(dy.float())
    assert_product_close(y, y_ref.detach(), "y", roundings=2)
    for got, ref, name in zip(leaves, ref_leaves, ("dx", "dw1", "dw2")):
        assert_product_close(got.grad, ref.grad, name, roundings=3)


def test_dsd_into_a_given_buffer(stk):
    """dsd(out=...) writes the same product into the caller's rows (a wider buffer's leading rows)."""
    np.random.seed(11)
    s = stk.random.randn((384, 256), 0.5, 128).to("cuda")
    b = (torch.randn(256, 512, device="cuda") * 0.1).half()
    with torch.no_grad():
        ref = stk.ops.dsd(s, b)
        buf = torch.full((640, 512), float("nan"), dtype=torch.float16, device="cuda")
        got = stk.ops.dsd(s, b, out=buf[:384])
        assert got.data_ptr() == buf.data_ptr() and torch.equal(got, ref)
        assert bool(torch.isnan(buf[384:]).all())
        with pytest.raises(ValueError):
            stk.ops.dsd(s, b, out=buf[:256])
    with pytest.raises(ValueError):
        stk.ops.dsd(s, b.clone().requires_grad_(True), out=buf[:384])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dmoe_shaped_products_full_size(stk, dtype):
    """BASELINE configs[1]-shaped problem at full size (T=16384, h=1024, f=4096, E=8): forward and
    the four backward products, checked per expert against dense fp32 products of the same 16-bit
    operands (identical math for a block-diagonal topology), plus two size-independent properties:
    linearity of DSD in the dense operand and SDD -> to_dense -> to_sparse round trip."""
    from stk_b200 import dmoe
    dev = "cuda"
    T, h, f, E = 16384, 1024, 4096, 8
    g = torch.Generator().manual_seed(0)
    ids = torch.multinomial(torch.full((E,), 1.0 / E), T, replacement=True, generator=g).to(dev)
    index, padded, bin_rows, total = dmoe.route_top1(ids, E)
    topo = dmoe.topology_from_bins(bin_rows, total // 128, f, dtype, dev)
    x = dmoe.permute_tokens((torch.randn(T, h, generator=g) * 0.02).to(dtype).to(dev), index, total)
    w1 = (torch.randn(h, E * f, generator=g) * 0.02).to(dtype).to(dev).requires_grad_(True)
    w2 = (torch.randn(E * f, h, generator=g) * 0.02).to(dtype).to(dev).requires_grad_(True)
    x.requires_grad_(True)
    hid = stk.ops.sdd(x, w1, topo)
    y = stk.ops.dsd(hid, w2)
    dy = (torch.randn(total, h, generator=g) * 0.02).to(dtype).to(dev)
    y.backward(dy)
    rows = (padded // 128).tolist()
    cpb = f // 128
    r0 = 0
    for e in range(E):
        nr = rows[e]
        if nr == 0:
            continue
        sl = slice(r0 * 128, (r0 + nr) * 128)
        xe = x.detach()[sl].float()
        w1e = w1.detach()[:, e * f:(e + 1) * f].float()
        w2e = w2.detach()[e * f:(e + 1) * f].float()
        he = hid.data.detach()[r0 * cpb:(r0 + nr) * cpb].view(nr, cpb, 128, 128).permute(0, 2, 1, 3).reshape(nr * 128, f)
        assert_product_close(he, xe @ w1e, f"sdd expert {e}")
        he32 = he.float()
        assert_product_close(y.detach()[sl], he32 @ w2e, f"dsd expert {e}")
        dye = dy[sl].float()
        assert_product_close(w2.grad[e * f:(e + 1) * f], he32.t() @ dye, f"dw2 expert {e}")     # dsd, S transposed
        dhe = dye @ w2e.t()                                                                       # sdd, rhs transposed
        assert_product_close(x.grad[sl], dhe.to(dtype).float() @ w1e.t(), f"dx expert {e}")       # dsd, rhs transposed
        assert_product_close(w1.grad[:, e * f:(e + 1) * f], xe.t() @ dhe.to(dtype).float(), f"dw1 expert {e}")  # dds
        r0 += nr
    with torch.no_grad():
        # linearity: dsd(S, a + b) == dsd(S, a) + dsd(S, b) up to output rounding
        a = (torch.randn(E * f, 256, generator=g) * 0.02).to(dtype).to(dev)
        b = (torch.randn(E * f, 256, generator=g) * 0.02).to(dtype).to(dev)
        lhs = stk.ops.dsd(hid, (a.float() + b.float()).to(dtype))
        rhs = stk.ops.dsd(hid, a).float() + stk.ops.dsd(hid, b).float()
        assert_product_close(lhs, rhs, "dsd linearity", roundings=3)
    del y, dy, x, w1, w2
    torch.cuda.empty_cache()


def test_dmoe_routing_kernels_match_host_logic(stk):
    """Sort by expert, padded-bin gather index, row gather / scatter and the closed-form topology on
    the GPU against the same steps done with torch indexing on the host and against the generic
    transpose kernel."""
    from stk_b200 import dmoe
    from tests.test_dmoe_host import check_routing
    g = torch.Generator().manual_seed(3)
    for tokens, experts, hidden in [(5000, 8, 64), (16384, 64, 256), (777, 3, 8)]:
        ids = torch.randint(0, experts, (tokens,), generator=g)
        if experts == 64:
            ids[ids == 5] = 6          # an expert without tokens
        x = torch.randn(tokens, hidden, generator=g).half()
        check_routing(dmoe, x.cuda(), ids.cuda(), experts)
        order_d, offsets_d = dmoe.sort_by_expert(ids.cuda(), experts)
        order_h, offsets_h = dmoe.sort_by_expert(ids, experts)
        assert torch.equal(order_d.cpu(), order_h) and torch.equal(offsets_d.cpu(), offsets_h)
        # received-rows layout of a 4-rank exchange: counts [peer, local expert]
        counts = torch.randint(0, 300, (4, experts // 1 if experts < 8 else 8), generator=g)
        total = int((((counts.sum(0) + 127) // 128) * 128).sum())
        idx_h, rows_h = dmoe.bin_index(counts, total)
        idx_d, rows_d = dmoe.bin_index(counts.cuda(), total)
        assert torch.equal(idx_d.cpu(), idx_h) and torch.equal(rows_d.cpu(), rows_h)
        recv = torch.randn(int(counts.sum()), hidden, generator=g).half()
        padded_d = dmoe.gather_rows(recv.cuda(), idx_d, total)
        assert torch.equal(padded_d.cpu(), dmoe.gather_rows(recv, idx_h, total))
        back = dmoe.scatter_rows(padded_d, idx_d, recv.shape[0])
        assert torch.equal(back.cpu(), recv)
        # closed-form topology == topology built from its row-major half by the transpose kernel
        topo = dmoe.topology_from_bins(rows_d, int(rows_h.sum()), 512, torch.float16, "cuda")
        ref = stk.Matrix(topo.size(), topo.data, topo.row_indices, topo.column_indices, topo.offsets)
        for key in META_KEYS:
            assert torch.equal(getattr(topo, key), getattr(ref, key)), key
        expect_rows = torch.repeat_interleave(torch.arange(int(rows_h.sum())), 4).to(torch.int16)
        assert torch.equal(topo.row_indices.cpu(), expect_rows)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sdd_with_fused_gelu(stk, dtype):
    """sdd_gelu == GeLU (exact erf form) of the fp32 product, rounded once."""
    np.random.seed(9)
    torch.manual_seed(9)
    topo = stk.random.mask(512, 768, 0.4, 128).to("cuda")
    r, c = topo.row_indices.cpu().numpy(), topo.column_indices.cpu().numpy()
    a = torch.randn(512, 192).to(dtype)
    b = torch.randn(192, 768).to(dtype)
    full = torch.nn.functional.gelu(a.float() @ b.float())
    blocks = full.reshape(4, 128, 6, 128).permute(0, 2, 1, 3)[torch.from_numpy(r).long(), torch.from_numpy(c).long()]
    out = stk.ops.sdd_gelu(a.cuda(), b.cuda(), topo)
    assert out.dtype == dtype and isinstance(out, stk.Matrix)
    assert_product_close(out.data, blocks, "sdd_gelu")
    # and it equals the unfused pipeline up to the extra rounding of the unfused one
    unfused = torch.nn.functional.gelu(stk.ops.sdd(a.cuda(), b.cuda(), topo).data.float())
    assert_product_close(out.data, unfused, "sdd_gelu vs sdd+gelu", roundings=2)
