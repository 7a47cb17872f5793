"""Per-product timing on the benchmark shapes other than the headline one:

    python -m stk_b200.benchmarks c3     # dMoE forward + backward products, 16 experts with Zipf token counts, bf16
    python -m stk_b200.benchmarks c4     # random block sparsity on 8192^3, bf16, all op / transpose combinations
    python -m stk_b200.benchmarks train  # forward + backward of the experts' MLP, fused against unfused

Every line: nonzero-block TFLOP/s (2 * nnz * 128 * 128 * dense extent / time) with the 128x128 kernel
forced, the 128x256 row kernel forced (DSD and DDS; SDD runs the 128x128 kernel in that column), the
CTA-pair kernel forced and the per-topology choice, against a cuBLAS GEMM (torch.matmul)
of the same useful FLOPs timed in the same run.  CUDA events around 20 back-to-back launches after 5
warm-up launches; operands (hundreds of MB) exceed the L2, which is not flushed.
"""
import sys

import numpy as np
import torch

import stk_b200 as stk
from stk_b200 import dmoe
from stk_b200.backend import kernels


def _time_ms(fn, iters=20, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    torch.cuda._sleep(10_000_000)      # the host runs ahead: launch latency is not timed
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def _report(name, flops, fn, dense_fn):
    saved, cells = kernels.PAIR_MODE, []
    try:
        for mode in ("0", "3", "1", "auto"):
            kernels.PAIR_MODE = mode
            cells.append(_time_ms(fn))
    finally:
        kernels.PAIR_MODE = saved
    dense = _time_ms(dense_fn)
    tf = lambda ms: flops / ms / 1e9
    print(f"| {name:24s} | {tf(cells[0]):5.0f} | {tf(cells[1]):5.0f} | {tf(cells[2]):5.0f} | {tf(cells[3]):5.0f} | "
          f"{cells[3] * 1e3:7.1f} | {tf(dense):5.0f} | {dense / cells[3]:4.2f} |", flush=True)


_HEADER = ("| product                  | 128x128 | 128x256 | pair | auto TFLOP/s | auto us | cuBLAS TFLOP/s | auto / cuBLAS |\n"
           "|---|---|---|---|---|---|---|---|")


def config3(dev="cuda"):
    T, h, f, E, dtype = 32768, 2048, 8192, 16, torch.bfloat16
    g = torch.Generator().manual_seed(0)
    p = (torch.arange(E) + 1.0) ** -1.2
    ids = torch.multinomial(p / p.sum(), T, replacement=True, generator=g).to(dev)
    _, padded, _, total = dmoe.route_top1(ids, E)
    topo = dmoe.block_diagonal_topology(padded, f, dtype, dev)
    nnz = topo.data.shape[0]
    print(f"dMoE fwd+bwd products, T={T} h={h} f={f} E={E} bf16; padded rows {total}, {nnz} blocks, "
          f"block rows per expert {(padded // 128).tolist()}")
    print(_HEADER)
    rand = lambda *shape: torch.empty(*shape, dtype=dtype, device=dev).normal_(0, 0.02)
    x, w1, w2, dy = rand(total, h), rand(h, E * f), rand(E * f, h), rand(total, h)
    hid = stk.ops.sdd(x, w1, topo)
    flops = 2.0 * nnz * 128 * 128 * h
    wa, wb, ha = w1[:, :f].contiguous(), w2[:f].contiguous(), rand(total, f)   # one expert's dense twin
    _report("fwd sdd   x @ w1", flops, lambda: stk.ops.sdd(x, w1, topo), lambda: x @ wa)
    _report("fwd dsd   h @ w2", flops, lambda: stk.ops.dsd(hid, w2), lambda: ha @ wb)
    _report("bwd sdd   dy @ w2^T", flops, lambda: stk.ops.sdd(dy, w2.t(), topo), lambda: dy @ wb.t())
    _report("bwd dsd   h^T @ dy", flops, lambda: stk.ops.dsd(hid.t(), dy), lambda: ha.t() @ dy)
    _report("bwd dsd   dh @ w1^T", flops, lambda: stk.ops.dsd(hid, w1.t()), lambda: ha @ wa.t())
    _report("bwd dds   x^T @ dh", flops, lambda: stk.ops.dds(x.t(), hid), lambda: x.t() @ ha)


def config4(dev="cuda"):
    M = N = K = 8192
    dtype = torch.bfloat16
    for density in (0.05, 0.125, 0.25, 0.5):
        np.random.seed(0)
        topo = stk.random.mask(M, N, 1 - density, 128).to(dev)
        nnz = topo.data.shape[0]
        s = stk.Matrix(topo.size(), torch.randn(nnz, 128, 128, device=dev).to(dtype), topo.row_indices,
                       topo.column_indices, topo.offsets, topo.column_indices_t, topo.offsets_t,
                       topo.block_offsets_t)
        a, b = torch.randn(M, K, device=dev).to(dtype), torch.randn(K, N, device=dev).to(dtype)
        flops = 2.0 * nnz * 128 * 128 * K
        nd = max(128, int(round(N * density / 128)) * 128)     # dense GEMM with the same FLOPs: 8192 x 8192 x nd
        bd = torch.randn(K, nd, device=dev).to(dtype)
        an, bn = a[:, :nd].contiguous(), b[:nd].contiguous()
        rows, cols, tiles, _, _ = kernels.pair_hints(topo.offsets, topo.row_indices, topo.column_indices, N // 128,
                                                     topo.offsets_t, topo.column_indices_t, need_t=True, wait=True)
        print(f"\nrandom topology 8192^2, density {density}: {nnz} blocks; useful share of the pair kernel's work: "
              f"row pairs {rows:.2f}, column pairs {cols:.2f}, 2x2 tiles {tiles:.2f}")
        print(_HEADER)
        _report("sdd  a @ b", flops, lambda: stk.ops.sdd(a, b, s), lambda: a @ bd)
        _report("sdd  a^T @ b^T", flops, lambda: stk.ops.sdd(a.t(), b.t(), s), lambda: a @ bd)
        _report("dsd  s @ b", flops, lambda: stk.ops.dsd(s, b), lambda: an @ bn)
        _report("dsd  s^T @ b", flops, lambda: stk.ops.dsd(s.t(), b), lambda: an @ bn)
        _report("dds  a @ s", flops, lambda: stk.ops.dds(a, s), lambda: a @ bd)
        _report("dds  a @ s^T", flops, lambda: stk.ops.dds(a, s.t()), lambda: a @ bd)


def single(density=0.25, dev="cuda"):
    """A few launches of s @ b and a @ s on one random topology, kernel chosen by STK_B200_PAIR_MODE:
    the small case for a profiler capture (python -m stk_b200.benchmarks single 0.25)."""
    M = N = K = 8192
    dtype = torch.bfloat16
    np.random.seed(0)
    topo = stk.random.mask(M, N, 1 - density, 128).to(dev)
    nnz = topo.data.shape[0]
    s = stk.Matrix(topo.size(), torch.randn(nnz, 128, 128, device=dev).to(dtype), topo.row_indices,
                   topo.column_indices, topo.offsets, topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
    a, b = torch.randn(M, K, device=dev).to(dtype), torch.randn(K, N, device=dev).to(dtype)
    flops = 2.0 * nnz * 128 * 128 * K
    for name, fn in (("dsd s @ b", lambda: stk.ops.dsd(s, b)), ("dds a @ s", lambda: stk.ops.dds(a, s)),
                     ("sdd a @ b", lambda: stk.ops.sdd(a, b, s))):
        ms = _time_ms(fn, iters=3, warm=2)
        print(f"{name}: {nnz} blocks, mode {kernels.PAIR_MODE}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.0f} TFLOP/s")


def train_step(dev="cuda"):
    """Forward + backward of the experts' MLP on the headline shape (T=16384, h=1024, f=4096, E=8, fp16):
    dmoe.expert_mlp (GeLU and its backward inside the products' epilogues) against
    sdd -> torch gelu -> dsd differentiated by autograd."""
    T, h, f, E, dtype = 16384, 1024, 4096, 8, torch.float16
    g = torch.Generator().manual_seed(0)
    ids = torch.multinomial(torch.full((E,), 1.0 / E), T, replacement=True, generator=g).to(dev)
    _, padded, _, total = dmoe.route_top1(ids, E)
    topo = dmoe.block_diagonal_topology(padded, f, dtype, dev)
    rand = lambda *shape: torch.empty(*shape, dtype=dtype, device=dev).normal_(0, 0.02).requires_grad_(True)
    x, w1, w2 = rand(total, h), rand(h, E * f), rand(E * f, h)
    dy = torch.empty(total, h, dtype=dtype, device=dev).normal_(0, 0.02)

    def unfused():
        hid = stk.ops.sdd(x, w1, topo)
        act = stk.Matrix(hid.size(), torch.nn.functional.gelu(hid.data), hid.row_indices, hid.column_indices,
                         hid.offsets, hid.column_indices_t, hid.offsets_t, hid.block_offsets_t)
        stk.ops.dsd(act, w2).backward(dy)

    def fused():
        dmoe.expert_mlp(x, w1, w2, topo).backward(dy)

    flops = 6 * 2.0 * topo.data.shape[0] * 128 * 128 * h          # two products forward, four backward
    for name, fn in (("sdd -> gelu -> dsd, autograd", unfused), ("dmoe.expert_mlp", fused)):
        ms = _time_ms(fn, iters=10, warm=3)
        print(f"{name:32s} fwd+bwd {ms * 1e3:7.1f} us  {flops / ms / 1e9:5.0f} TFLOP/s")


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "c3"
    if which == "train":
        train_step()
    else:
        with torch.no_grad():
            if which == "single":
                single(float(sys.argv[2]) if len(sys.argv) > 2 else 0.25)
            else:
                {"c3": config3, "c4": config4}[which]()
