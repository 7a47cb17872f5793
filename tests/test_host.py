"""CPU-only tests: the C ABI exports what the header declares, and the host-side classes behave
like the reference's (no kernel is launched here)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import stk_oracle as oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "stk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(stk_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from stk_b200.backend import lib
    names = _declared_functions()
    assert len(names) >= 14
    cdll = ctypes.CDLL(lib.LIB_PATH)
    for name in names:
        assert hasattr(cdll, name), f"{name} declared in include/stk_b200.h but not exported"
    assert sorted(lib.SIGNATURES) == names, "ctypes signatures out of sync with the header"
    loaded = lib.load()
    assert loaded.stk_b200_version() == 100
    assert lib.error_string(0) == "ok"
    assert "dimension" in lib.error_string(-2)


def test_argument_validation_happens_before_any_launch():
    """Bad arguments are rejected by the C entry points on the host (no GPU needed)."""
    from stk_b200.backend import lib
    l = lib.load()
    null = ctypes.c_void_p(0)
    # M not a multiple of 128 / K not a multiple of 32 / bad dtype
    assert l.stk_b200_sdd(null, null, null, null, null, null, 100, 128, 128, 1, 0, 128, 0, 128, 0, 0, 0, null, null, null) == -2
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 48, 1, 0, 128, 0, 128, 0, 0, 0, null, null, null) == -2
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 128, 1, 0, 128, 0, 128, 7, 0, 0, null, null, null) == -3
    # nnz == 0 is a no-op for SDD even with NULL pointers
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 128, 0, 0, 128, 0, 128, 0, 1, 0, null, null, null) == 0
    # NULL operands
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 128, 1, 0, 128, 0, 128, 0, 0, 0, null, null, null) == -1
    # an epilogue with an auxiliary tensor needs one; unknown epilogue codes are rejected
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 128, 1, 0, 128, 0, 128, 0, 0, 2, null, null, null) == -1
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 128, 1, 0, 128, 0, 128, 0, 0, 4, null, null, null) == -2
    assert l.stk_b200_dsd(null, null, null, null, null, null, 128, 128, 100, 1, 0, 0, 128, 128, 0, 0, null, null) == -2
    assert l.stk_b200_transpose_meta(null, null, -1, 4, null, null, null, null, 0, null) == -2
    assert l.stk_b200_transpose_meta(null, null, 4, 40000, null, null, null, null, 0, null) == -9
    assert l.stk_b200_block_mask(null, 8, 8, 8, 3, 2, null, null) == -2
    assert l.stk_b200_block_mask(null, 8, 8, 8, 8, 3, null, null) == -3
    assert l.stk_b200_to_dense(null, null, null, 2, 2, 8, 8, null, 16, null) == -3
    # regroup_blocks: blockings 16 / 32 / 64, element sizes 1 / 2 / 4, aligned buffers
    assert l.stk_b200_regroup_blocks(null, null, null, 4, 1, 48, 2, 1, null) == -2
    assert l.stk_b200_regroup_blocks(null, null, null, 4, 1, 128, 2, 1, null) == -2
    assert l.stk_b200_regroup_blocks(null, null, null, 4, 1, 64, 3, 1, null) == -3
    assert l.stk_b200_regroup_blocks(null, null, null, 0, 0, 64, 2, 1, null) == 0
    assert l.stk_b200_regroup_blocks(null, null, null, 4, 1, 64, 2, 1, null) == -1
    assert l.stk_b200_regroup_blocks(ctypes.c_void_p(8), ctypes.c_void_p(16), ctypes.c_void_p(16), 4, 1, 64, 2, 1, null) == -4
    # workspace sizing: small problems need none, large ones a bounded amount
    ws = l.stk_b200_transpose_meta_workspace_bytes
    assert ws(16, 8) == 0 and ws(0, 100) == 0
    assert 0 < ws(241645, 7168) <= 4 << 20
    with pytest.raises(ValueError):
        lib.check(-2, "x")
    with pytest.raises(RuntimeError):
        lib.check(-6, "x")


def _c1_matrix(stk):
    np.random.seed(0)
    m = oracle.mask(1024, 1024, 0.75, 128)
    t = lambda k: torch.from_numpy(m[k])
    return stk.Matrix(torch.Size((1024, 1024)), m["data"], t("row_indices"), t("column_indices"),
                      t("offsets"), t("column_indices_t"), t("offsets_t"), t("block_offsets_t"))


def test_matrix_api_mirrors_reference():
    import stk_b200 as stk
    m = _c1_matrix(stk)
    m.validate()
    assert m.blocking == 128 and m.nnz == 16 * 128 * 128 and m.dim() == 2
    assert m.shape == m.size() == torch.Size((1024, 1024))
    assert m.is_contiguous() and not m.is_cuda and m.dtype == torch.float16
    t = m.t()
    assert not t.is_contiguous() and t.t().is_contiguous()
    assert t.data.data_ptr() == m.data.data_ptr()          # O(1) view, nothing copied
    assert t.block_offsets_t.data_ptr() == m.block_offsets_t.data_ptr()
    with pytest.raises(ValueError):
        m.contiguous()
    c = m.clone()
    assert c.data.data_ptr() != m.data.data_ptr() and torch.equal(c.offsets_t, m.offsets_t)
    b = m.clone().to(torch.bfloat16)                        # values converted, metadata untouched
    assert b.dtype == torch.bfloat16 and b.row_indices.dtype == torch.int16 and b.offsets.dtype == torch.int32
    b.validate()
    with pytest.raises(ValueError):
        m.clone().to(torch.float32)
    v = m.view(2, 512, 1024)
    assert v.dim() == 3 and v.size() == (2, 512, 1024)
    with pytest.raises(ValueError):
        v.t()
    with pytest.raises(ValueError):
        m.view(2048, 512)
    m.requires_grad_(True)
    assert m.requires_grad
    (m.data.float().sum() * 2).backward()
    g = m.grad
    assert isinstance(g, stk.Matrix) and g.is_contiguous() and bool((g.data == 2).all())
    assert not m.t().grad.is_contiguous()
    prod = stk.ops.mul(m, m)
    assert isinstance(prod, stk.Matrix) and prod.offsets_t.data_ptr() == m.offsets_t.data_ptr()
    assert stk.ops.sum(ones_small := stk.ops.mul(m, m)).dtype == torch.float16  # fp16 sum, as in the reference
    ones = stk.ops.ones_like(m)
    assert bool((ones.data == 1).all()) and ones.column_indices_t.data_ptr() == m.column_indices_t.data_ptr()


def test_matrix_validation_errors():
    import stk_b200 as stk
    m = _c1_matrix(stk)
    f = dict(size=m.size(), data=m.data, row_indices=m.row_indices, column_indices=m.column_indices,
             offsets=m.offsets, column_indices_t=m.column_indices_t, offsets_t=m.offsets_t,
             block_offsets_t=m.block_offsets_t)

    def build(**kw):
        return stk.Matrix(**{**f, **kw})

    with pytest.raises(ValueError):
        build(data=m.data.float()).validate()
    with pytest.raises(ValueError):
        build(row_indices=m.row_indices.int()).validate()
    with pytest.raises(ValueError):
        build(offsets=m.offsets.long()).validate()
    with pytest.raises(ValueError):
        build(offsets=m.offsets[:-1]).validate()
    with pytest.raises(ValueError):
        build(size=torch.Size((1000, 1024))).validate()
    with pytest.raises(ValueError):
        build(data=m.data[:, :, :64]).validate()
    with pytest.raises(ValueError):   # 16-bit indices cannot address this many block columns
        build(size=torch.Size((1024, 32768 * 128)))
    build(data=m.data.bfloat16()).validate()   # bf16 values are accepted (reference: fp16 only)


def test_linear_ops_type_checks_and_no_cpu_path():
    import stk_b200 as stk
    m = _c1_matrix(stk)
    x = torch.zeros(1024, 128, dtype=torch.float16)
    with pytest.raises(AssertionError):
        stk.ops.dsd(x, x)
    with pytest.raises(AssertionError):
        stk.ops.dds(m, m)
    with pytest.raises(AssertionError):
        stk.ops.sdd(x, x, m.t())
    with pytest.raises(RuntimeError, match="no CPU path|CUDA"):
        stk.ops.dsd(m, x)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            stk.ops.to_sparse(torch.ones(8, 8, dtype=torch.float16), 1)


def test_dense_mask_matches_oracle_pattern():
    import stk_b200 as stk
    for rows, cols, sparsity, blocking, seed in [(8, 16, 0.5, 1, 1), (128, 256, 0.5, 16, 2),
                                                 (512, 512, 0.875, 128, 3)]:
        np.random.seed(seed)
        mine = stk.random.dense_mask(rows, cols, sparsity, blocking)
        np.random.seed(seed)
        ref = oracle.dense_mask(rows, cols, sparsity, blocking)
        assert mine.dtype == torch.float32 and torch.equal(mine, ref)


def test_autograd_wiring_matches_dense_calculus(monkeypatch):
    """The backward formulas, with the CUDA launchers replaced by dense stand-ins on the host:
    every gradient of dsd / dds / sdd in every transpose combination equals torch autograd's."""
    import stk_b200 as stk
    from stk_b200.backend import sputnik

    def densify(shape, data, row_idx, col_idx, transposed):
        storage = (shape[1], shape[0]) if transposed else tuple(shape)
        d = oracle.to_dense(data.detach(), row_idx.numpy(), col_idx.numpy(), storage)
        return d.t() if transposed else d

    def fake_dsd(shape, data, offsets, row_idx, col_idx, offsets_t, col_idx_t, blk_t, transpose_a, rhs, out):
        out.copy_(densify(shape, data, row_idx, col_idx, transpose_a).double() @ rhs.double())

    def fake_dds(lhs, shape, data, offsets, row_idx, col_idx, offsets_t, col_idx_t, blk_t, transpose_b, out):
        out.copy_(lhs.double() @ densify(shape, data, row_idx, col_idx, transpose_b).double())

    def fake_sdd(lhs, rhs, shape, out, offsets, row_idx, col_idx):
        full = lhs.double() @ rhs.double()
        b = out.shape[1]
        blocks = full.reshape(shape[0] // b, b, shape[1] // b, b).permute(0, 2, 1, 3)
        out.copy_(blocks[row_idx.long(), col_idx.long()])

    monkeypatch.setattr(sputnik.backend, "dsd", fake_dsd)
    monkeypatch.setattr(sputnik.backend, "dds", fake_dds)
    monkeypatch.setattr(sputnik.backend, "sdd", fake_sdd)

    np.random.seed(11)
    torch.manual_seed(11)
    b = 4
    pat = oracle.block_pattern(12, 8, 0.5, b)
    r, c = np.nonzero(pat)
    offsets = np.concatenate([[0], np.cumsum(pat.sum(1))]).astype(np.int32)
    cit, offt, bot = oracle.transpose(8 // b, r.astype(np.int16), c.astype(np.int16))

    def sparse(values):
        return stk.Matrix(torch.Size((12, 8)), values, torch.from_numpy(r.astype(np.int16)),
                          torch.from_numpy(c.astype(np.int16)), torch.from_numpy(offsets),
                          torch.from_numpy(cit), torch.from_numpy(offt), torch.from_numpy(bot))

    mask = torch.from_numpy(np.kron(pat, np.ones((b, b)))).double()
    for ts in (False, True):
        for td in (False, True):
            vals = torch.randn(len(r), b, b, dtype=torch.double, requires_grad=True)
            s = sparse(vals)
            s_dense = oracle.to_dense(vals.detach(), r, c, (12, 8)).requires_grad_(True)
            S, SD = (s.t(), s_dense.t()) if ts else (s, s_dense)
            # dsd: op(S) [.., K] @ D [K, 5]
            kdim = SD.shape[1]
            d_store = torch.randn((5, kdim) if td else (kdim, 5), dtype=torch.double)
            d1 = d_store.clone().requires_grad_(True)
            d2 = d_store.clone().requires_grad_(True)
            out = stk.ops.dsd(S, d1.t() if td else d1)
            ref = SD @ (d2.t() if td else d2)
            w = torch.randn_like(ref)
            (out * w).sum().backward()
            (ref * w).sum().backward()
            torch.testing.assert_close(out, ref)
            torch.testing.assert_close(d1.grad, d2.grad)
            torch.testing.assert_close(oracle.to_dense(vals.grad, r, c, (12, 8)), s_dense.grad * mask)
            # dds: D [5, K] @ op(S) [K, ..]
            vals.grad = None
            s_dense.grad = None
            kdim = SD.shape[0]
            d_store = torch.randn((kdim, 5) if td else (5, kdim), dtype=torch.double)
            d1 = d_store.clone().requires_grad_(True)
            d2 = d_store.clone().requires_grad_(True)
            out = stk.ops.dds(d1.t() if td else d1, S)
            ref = (d2.t() if td else d2) @ SD
            w = torch.randn_like(ref)
            (out * w).sum().backward()
            (ref * w).sum().backward()
            torch.testing.assert_close(out, ref)
            torch.testing.assert_close(d1.grad, d2.grad)
            torch.testing.assert_close(oracle.to_dense(vals.grad, r, c, (12, 8)), s_dense.grad * mask)
    # sdd: A [12, 6] @ B [6, 8] on the topology
    topo = sparse(torch.zeros(len(r), b, b, dtype=torch.double))
    for ta in (False, True):
        for tb in (False, True):
            a_store = torch.randn((6, 12) if ta else (12, 6), dtype=torch.double)
            b_store = torch.randn((8, 6) if tb else (6, 8), dtype=torch.double)
            a1, a2 = (a_store.clone().requires_grad_(True) for _ in range(2))
            b1, b2 = (b_store.clone().requires_grad_(True) for _ in range(2))
            out = stk.ops.sdd(a1.t() if ta else a1, b1.t() if tb else b1, topo)
            ref = ((a2.t() if ta else a2) @ (b2.t() if tb else b2)) * mask
            w = torch.randn(12, 8, dtype=torch.double)
            w_blocks = w.reshape(3, b, 2, b).permute(0, 2, 1, 3)[r, c]
            (out.data * w_blocks).sum().backward()
            (ref * w).sum().backward()
            torch.testing.assert_close(oracle.to_dense(out.data.detach(), r, c, (12, 8)), ref.detach())
            torch.testing.assert_close(a1.grad, a2.grad)
            torch.testing.assert_close(b1.grad, b2.grad)


def test_products_reject_mixed_dtypes_and_unknown_kernel_modes():
    """float16 and bfloat16 operands in one product would be reinterpreted bit for bit: the launchers
    refuse them before anything else (no GPU needed).  pair_mode values outside 0..3 are
    rejected by the C entry points."""
    from stk_b200.backend import kernels, lib
    h = lambda *shape: torch.zeros(*shape, dtype=torch.float16)
    b = lambda *shape: torch.zeros(*shape, dtype=torch.bfloat16)
    idx = torch.zeros(1, dtype=torch.int16)
    off = torch.zeros(2, dtype=torch.int32)
    blk = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(ValueError, match="share one dtype"):
        kernels.dsd((128, 128), h(1, 128, 128), off, idx, idx, off, idx, blk, False, b(128, 128), b(128, 128))
    with pytest.raises(ValueError, match="share one dtype"):
        kernels.dds(h(128, 128), (128, 128), b(1, 128, 128), off, idx, idx, off, idx, blk, False, h(128, 128))
    with pytest.raises(ValueError, match="share one dtype"):
        kernels.sdd(h(128, 128), b(128, 128), (128, 128), h(1, 128, 128), off, idx, idx)
    l = lib.load()
    null = ctypes.c_void_p(0)
    assert l.stk_b200_sdd(null, null, null, null, null, null, 128, 128, 128, 1, 0, 128, 0, 128, 0, 4, 0, null, null, null) == -2
    assert l.stk_b200_dsd(null, null, null, null, null, null, 128, 128, 128, 1, 0, 0, 128, 128, 0, 7, null, null) == -2
    assert l.stk_b200_pair_plan(null, null, 0, null, 0, null) == -2
    assert l.stk_b200_pair_plan(null, null, 4, null, 0, null) == -1
    assert l.stk_b200_pair_plan_bytes(100) == 4 * 204
    assert l.stk_b200_ep_barrier(null, 2, 0, 1, 100, null) == -1
    assert l.stk_b200_ep_plan(null, 2, 8, 0, 128, 1, null, null, null, null) == -1
    assert l.stk_b200_weighted_sum_rows(null, null, null, null, 4, 2, 24, 0, null) == -2


def test_matrix_accepts_int32_block_indices():
    """validate() takes int16 or int32 block indices, but not a mix of the two."""
    import stk_b200 as stk
    data = torch.zeros((1, 8, 8), dtype=torch.float16)
    off = torch.tensor([0, 1], dtype=torch.int32)
    i16, i32 = torch.zeros(1, dtype=torch.int16), torch.zeros(1, dtype=torch.int32)
    full = lambda r, c: stk.Matrix(torch.Size((8, 8)), data, r, c, off, r, off, torch.zeros(1, dtype=torch.int32))
    full(i16, i16).validate()
    full(i32, i32).validate()
    with pytest.raises(ValueError, match="one integer type"):
        full(i16, i32).validate()
    with pytest.raises(ValueError, match="int16 or int32"):
        full(i32.long(), i32.long()).validate()


def test_float8_entry_points_check_their_arguments():
    """dtype 2 (float8 e4m3 operands): rows of 8-bit operands start on 16-byte boundaries, the 128x256
    kernels and the training epilogues do not take part, and the Python launchers refuse mixed operand
    types before anything runs."""
    from stk_b200.backend import kernels, lib
    l = lib.load()
    null, fake = ctypes.c_void_p(0), ctypes.c_void_p(1 << 20)
    # a leading dimension that is not a multiple of 16 elements
    assert l.stk_b200_sdd(fake, fake, fake, fake, fake, fake, 128, 128, 128, 1, 0, 136, 1, 128, 2, 0, 0, null, null, null) == -4
    assert l.stk_b200_dsd(fake, fake, fake, fake, fake, fake, 128, 128, 128, 1, 0, 0, 136, 128, 2, 0, null, null) == -4
    # the 128x256 kernels are 16-bit only; no auxiliary tensor with 8-bit operands
    assert l.stk_b200_dsd(fake, fake, fake, fake, fake, fake, 128, 256, 128, 1, 0, 1, 128, 256, 2, 3, null, null) == -3
    assert l.stk_b200_sdd(fake, fake, fake, fake, fake, fake, 128, 128, 128, 1, 0, 128, 1, 128, 2, 0, 2, fake, null, null) == -2
    f8 = lambda *shape: torch.zeros(*shape).to(torch.float8_e4m3fn)
    h = lambda *shape: torch.zeros(*shape, dtype=torch.float16)
    idx = torch.zeros(1, dtype=torch.int16)
    off = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(ValueError, match="float8_e4m3fn operands go with"):
        kernels.sdd(f8(128, 128), h(128, 128), (128, 128), h(1, 128, 128), off, idx, idx)
    with pytest.raises(ValueError, match="float8_e4m3fn operands go with"):
        kernels.sdd(f8(128, 128), f8(128, 128), (128, 128), h(1, 128, 128), off, idx, idx)


def test_wide_shape_is_chosen_by_list_length_and_rounds(monkeypatch):
    """kernels._pair_shape: the 256x512 shape needs long lists (48 blocks on average) and a tail of
    rounds that does not eat its gain; forced modes override; only pair-kernel products are asked."""
    from stk_b200.backend import kernels
    monkeypatch.setattr(kernels, "_pairs_resident", lambda device: 74)
    monkeypatch.setattr(kernels, "PAIR_MODE", "auto")
    dev = torch.device("cpu")
    lists = 260                                            # block rows of a dMoE shard: 130 list pairs
    assert kernels._pair_shape(1, 112 * lists, lists, 4096, dev) == 2      # 130 * 8 = 1040 items, long lists
    assert kernels._pair_shape(1, 40 * lists, lists, 4096, dev) == 1       # lists too short
    assert kernels._pair_shape(1, 112 * lists, lists, 2048, dev) == 1      # 520 items: 7.03 rounds cost 8
    assert kernels._pair_shape(1, 112 * 136, 136, 4096, dev) == 1          # 544 items: 7.35 rounds cost 8
    assert kernels._pair_shape(1, 112 * 146, 146, 4096, dev) == 2          # 584 items: 7.9 rounds cost 8
    assert kernels._pair_shape(3, 112 * lists, lists, 4096, dev) == 3      # not a pair-kernel product
    assert kernels._pair_shape(0, 112 * lists, lists, 4096, dev) == 0
    monkeypatch.setattr(kernels, "PAIR_MODE", "2")
    assert kernels._pair_shape(1, 8 * lists, lists, 256, dev) == 2
    monkeypatch.setattr(kernels, "PAIR_MODE", "1")
    assert kernels._pair_shape(1, 112 * lists, lists, 4096, dev) == 1


def test_nvtx_wrapper_passes_calls_through(monkeypatch):
    """lib._Traced (STK_B200_NVTX=1) wraps launching entry points in an NVTX range and leaves their
    arguments and results alone; size queries and status reads are not wrapped."""
    from stk_b200.backend import lib
    raw = lib.load()
    raw = getattr(raw, "_lib", raw)
    events = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: events.append(("pop",)))
    traced = lib._Traced(raw)
    assert traced.stk_b200_pair_plan_bytes(100) == 4 * 204 and events == []
    null = ctypes.c_void_p(0)
    assert traced.stk_b200_pair_plan(null, null, 0, null, 0, null) == -2
    assert events == [("push", "stk_b200_pair_plan"), ("pop",)]


def test_small_block_products_refuse_what_they_cannot_regroup():
    """Blockings other than 16 / 32 / 64 / 128, and sparse shapes that are not multiples of 128, are refused
    on the host before anything runs."""
    import stk_b200 as stk
    from stk_b200.backend import kernels
    from stk_b200.ops import small_blocks

    def matrix(rows, cols, blocking):
        idx = torch.zeros(1, dtype=torch.int16)
        off = torch.zeros(rows // blocking + 1, dtype=torch.int32)
        off[1:] = 1
        off_t = torch.zeros(cols // blocking + 1, dtype=torch.int32)
        off_t[1:] = 1
        return stk.Matrix(torch.Size((rows, cols)), torch.ones(1, blocking, blocking, dtype=torch.float16), idx, idx.clone(),
                          off, idx.clone(), off_t, torch.zeros(1, dtype=torch.int32))

    with pytest.raises(kernels.DimensionError):
        small_blocks.coarse_topology(matrix(256, 256, 8))
    with pytest.raises(kernels.DimensionError):
        small_blocks.coarse_topology(matrix(192, 256, 64))
    with pytest.raises(kernels.DimensionError):
        stk.ops.dsd(matrix(256, 320, 64).t(), torch.zeros(256, 128, dtype=torch.float16))
