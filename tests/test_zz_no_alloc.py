"""The allocation-free transpose entry point (stk_b200_transpose_meta_static).

Some callers of this library cannot obtain device memory when they need the transposed metadata
(code that runs where the framework's allocator must not be re-entered, or a binding that can only
pass through the buffers it was handed).  For them the library carries its scratch counters in a
fixed array of its own.  This test drives that entry point through the C ABI, twice in a row on
different topologies - the array is shared and keeps the previous call's contents - and requires
bit-identical results to the ordinary entry point.  The file name sorts last so that it runs after
every other test; it also passes on its own in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _topology(block_rows, block_cols, density, seed):
    rng = np.random.default_rng(seed)
    r, c = np.nonzero(rng.random((block_rows, block_cols)) < density)
    return (torch.from_numpy(r.astype(np.int16)).cuda(), torch.from_numpy(c.astype(np.int16)).cuda())


def _outputs(nnz, block_cols):
    return (torch.empty(nnz, dtype=torch.int16, device="cuda"),
            torch.empty(block_cols + 1, dtype=torch.int32, device="cuda"),
            torch.empty(nnz, dtype=torch.int32, device="cuda"))


def test_static_scratch_entry_matches_workspace_entry():
    from stk_b200.backend import lib
    L = lib.load()
    stream = lib.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    # both topologies take the multi-kernel path (more than 1536 block columns / 32768 blocks),
    # the second one reuses counters the first one left non-zero
    for block_rows, block_cols, density, seed in [(96, 4096, 0.2, 1), (700, 2048, 0.05, 2),
                                                  (64, 8192, 0.1, 3)]:
        rows, cols = _topology(block_rows, block_cols, density, seed)
        nnz = rows.numel()
        ws_bytes = L.stk_b200_transpose_meta_workspace_bytes(nnz, block_cols)
        assert ws_bytes > 0, "case must exercise the scratch-using path"
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        expect = _outputs(nnz, block_cols)
        lib.check(L.stk_b200_transpose_meta(lib.ptr(rows), lib.ptr(cols), nnz, block_cols,
                                            *(lib.ptr(t) for t in expect), lib.ptr(ws), ws_bytes,
                                            stream), "stk_b200_transpose_meta")
        got = _outputs(nnz, block_cols)
        lib.check(L.stk_b200_transpose_meta_static(lib.ptr(rows), lib.ptr(cols), nnz, block_cols,
                                                   *(lib.ptr(t) for t in got), stream),
                  "stk_b200_transpose_meta_static")
        torch.cuda.synchronize()
        for a, b in zip(got, expect):
            assert torch.equal(a, b)
        # and both agree with a stable sort by column
        order = torch.argsort(cols.long(), stable=True)
        assert torch.equal(got[2].long(), order) and torch.equal(got[0], rows[order])
    # sizes beyond the built-in scratch are refused, nothing is launched
    null = ctypes.c_void_p(0)
    assert L.stk_b200_transpose_meta_static(null, null, 10, 8193, null, null, null, stream) == -9
    assert L.stk_b200_transpose_meta_static(null, null, (1 << 20) + 1, 64, null, null, null, stream) == -9
    assert "beyond" in lib.error_string(-9)
    assert lib.device_status() == 0
