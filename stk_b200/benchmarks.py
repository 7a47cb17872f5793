"""Per-product and per-kernel timing on the benchmark shapes other than the headline one:

    python -m stk_b200.benchmarks c2     # dMoE forward + backward products, 16 experts with Zipf token counts, bf16
    python -m stk_b200.benchmarks c3     # random block sparsity on 8192^3, bf16, all op / transpose combinations
    python -m stk_b200.benchmarks meta   # metadata / conversion / row-movement kernels: achieved GB/s
    python -m stk_b200.benchmarks train  # forward + backward of the experts' MLP, fused against unfused
    python -m stk_b200.benchmarks ref    # the reference's own Triton kernels on this GPU (needs oracle/_ref)
    python -m stk_b200.benchmarks single 0.25   # a few launches on one random topology (profiler case)

Products: nonzero-block TFLOP/s (2 * nnz * 128 * 128 * dense extent / time) with the 128x128 kernel
forced, the 128x256 row kernel forced, the CTA-pair kernel forced and the per-topology choice, against
a cuBLAS GEMM (torch.matmul) of the same useful FLOPs.  The candidates of one line are timed
INTERLEAVED (A, B, C, A, B, C, ... a few launches each, median over the rounds), so that the clock
drift of a GPU that warms up during the run hits all of them alike.  Operands (hundreds of MB) exceed
the L2, which is not flushed.  bench.py calls products_c2 / products_c3 / meta_kernels for the extra
keys of its JSON line.
"""
import os
import statistics
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


def time_interleaved(fns, rounds=5, iters=4, warm=2):
    """{name: median ms per call}: every round times `iters` back-to-back calls of each candidate in
    turn, so slow clock drift affects all candidates equally."""
    for fn in fns.values():
        for _ in range(warm):
            fn()
    samples = {name: [] for name in fns}
    for _ in range(rounds):
        for name, fn in fns.items():
            torch.cuda.synchronize()
            torch.cuda._sleep(2_000_000)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(iters):
                fn()
            stop.record()
            torch.cuda.synchronize()
            samples[name].append(start.elapsed_time(stop) / iters)
    return {name: statistics.median(v) for name, v in samples.items()}


def _with_mode(mode, fn):
    def run():
        saved = kernels.PAIR_MODE
        kernels.PAIR_MODE = mode
        try:
            return fn()
        finally:
            kernels.PAIR_MODE = saved
    return run


def _product_line(name, flops, fn, dense_fn, all_modes):
    """One product against its same-FLOP dense GEMM; all_modes adds the four forced kernels."""
    fns = {"auto": _with_mode("auto", fn), "cublas": dense_fn}
    if all_modes:
        fns.update({"tile128": _with_mode("0", fn), "row256": _with_mode("3", fn), "pair256": _with_mode("1", fn),
                    "wide512": _with_mode("2", fn)})
    fn()                                   # settles the kernel choice of an unknown topology
    torch.cuda.synchronize()
    fn()
    ms = time_interleaved(fns)
    tf = lambda t: round(flops / t / 1e9, 1)
    line = {"product": name, "tflops": tf(ms["auto"]), "us": round(ms["auto"] * 1e3, 1),
            "cublas_tflops": tf(ms["cublas"]), "vs_cublas": round(ms["cublas"] / ms["auto"], 3)}
    if all_modes:
        line.update({k: tf(ms[k]) for k in ("tile128", "row256", "pair256", "wide512")})
    return line


def _print_table(title, lines):
    print(title)
    modes = "tile128" in lines[0]
    head = "| product | " + ("128x128 | 128x256 | pair 256x256 | pair 256x512 (sdd: 256x256) | " if modes else "") + "auto TFLOP/s | auto us | cuBLAS TFLOP/s | auto / cuBLAS |"
    print(head)
    print("|" + "---|" * (head.count("|") - 1))
    for ln in lines:
        mid = f"{ln['tile128']:.0f} | {ln['row256']:.0f} | {ln['pair256']:.0f} | {ln['wide512']:.0f} | " if modes else ""
        print(f"| {ln['product']} | {mid}{ln['tflops']:.0f} | {ln['us']:.1f} | {ln['cublas_tflops']:.0f} | {ln['vs_cublas']:.2f} |",
              flush=True)


def products_c2(dev="cuda", all_modes=False):
    """The six products of a dMoE forward + backward pass (T=32768, h=2048, f=8192, E=16, Zipf(1.2)
    token counts, bf16): sdd NN, dsd N, sdd NT, dsd with S transposed, dsd with the dense operand
    transposed, dds with the dense operand transposed."""
    T, h, f, E, dtype = 32768, 2048, 8192, 16, torch.bfloat16
    g = torch.Generator().manual_seed(0)
    p = (torch.arange(E) + 1.0) ** -1.2
    ids = torch.multinomial(p / p.sum(), T, replacement=True, generator=g).to(dev)
    _, padded, _, total = dmoe.route_top1(ids, E)
    topo = dmoe.block_diagonal_topology(padded, f, dtype, dev)
    nnz = topo.data.shape[0]
    rand = lambda *shape: torch.empty(*shape, dtype=dtype, device=dev).normal_(0, 0.02)
    x, w1, w2, dy = rand(total, h), rand(h, E * f), rand(E * f, h), rand(total, h)
    hid = stk.ops.sdd(x, w1, topo)
    flops = 2.0 * nnz * 128 * 128 * h
    wa, wb, ha = w1[:, :f].contiguous(), w2[:f].contiguous(), rand(total, f)   # one expert's dense twin
    specs = [("fwd sdd x@w1", lambda: stk.ops.sdd(x, w1, topo), lambda: x @ wa),
             ("fwd dsd h@w2", lambda: stk.ops.dsd(hid, w2), lambda: ha @ wb),
             ("bwd sdd dy@w2^T", lambda: stk.ops.sdd(dy, w2.t(), topo), lambda: dy @ wb.t()),
             ("bwd dsd h^T@dy", lambda: stk.ops.dsd(hid.t(), dy), lambda: ha.t() @ dy),
             ("bwd dsd dh@w1^T", lambda: stk.ops.dsd(hid, w1.t()), lambda: ha @ wa.t()),
             ("bwd dds x^T@dh", lambda: stk.ops.dds(x.t(), hid), lambda: x.t() @ ha)]
    lines = [_product_line(n, flops, fn, dfn, all_modes) for n, fn, dfn in specs]
    info = {"padded_rows": total, "blocks": nnz, "block_rows_per_expert": (padded // 128).tolist()}
    return info, lines


def products_c3(dev="cuda", all_modes=False, densities=(0.05, 0.125, 0.25, 0.5)):
    """Random block sparsity on 8192^3, bf16: SDD NN / TT, DSD with S and S^T, DDS with S and S^T at
    every density, each against a dense GEMM of the same useful FLOPs."""
    M = N = K = 8192
    dtype = torch.bfloat16
    out = {}
    a, b = torch.randn(M, K, device=dev).to(dtype), torch.randn(K, N, device=dev).to(dtype)
    for density in densities:
        np.random.seed(0)
        topo = stk.random.mask(M, N, 1 - density, 128).to(dev)
        nnz = topo.data.shape[0]
        s = stk.Matrix(topo.size(), torch.randn(nnz, 128, 128, device=dev).to(dtype), topo.row_indices,
                       topo.column_indices, topo.offsets, topo.column_indices_t, topo.offsets_t,
                       topo.block_offsets_t)
        flops = 2.0 * nnz * 128 * 128 * K
        nd = max(128, int(round(N * density / 128)) * 128)     # dense GEMM with the same FLOPs: 8192 x 8192 x nd
        bd = torch.randn(K, nd, device=dev).to(dtype)
        an, bn = a[:, :nd].contiguous(), b[:nd].contiguous()
        specs = [("sdd a@b", lambda: stk.ops.sdd(a, b, s), lambda: a @ bd),
                 ("sdd a^T@b^T", lambda: stk.ops.sdd(a.t(), b.t(), s), lambda: a @ bd),
                 ("dsd s@b", lambda: stk.ops.dsd(s, b), lambda: an @ bn),
                 ("dsd s^T@b", lambda: stk.ops.dsd(s.t(), b), lambda: an @ bn),
                 ("dds a@s", lambda: stk.ops.dds(a, s), lambda: a @ bd),
                 ("dds a@s^T", lambda: stk.ops.dds(a, s.t()), lambda: a @ bd)]
        out[f"{density:g}"] = {"blocks": nnz, "lines": [_product_line(n, flops, fn, dfn, all_modes) for n, fn, dfn in specs]}
        del s, bd, an, bn
    return out


def meta_kernels(dev="cuda", peak_gbs=None):
    """Achieved GB/s of the metadata, conversion and row-movement kernels: algorithmic bytes (what the
    step must read and write at least) over the CUDA-event time of the calls that make it up."""
    from stk_b200.backend import lib
    results = []

    def add(name, nbytes, fn, note=""):
        ms = _time_ms(fn, iters=10, warm=3)
        gbs = nbytes / ms / 1e6
        results.append({"kernel": name, "algorithmic_mb": round(nbytes / 1e6, 3), "us": round(ms * 1e3, 1),
                        "gbs": round(gbs, 1), "frac": None if peak_gbs is None else round(gbs / peak_gbs, 3),
                        "note": note})

    dtype = torch.bfloat16
    for blocking in (128, 32, 16):
        M = N = 8192
        np.random.seed(1)
        R = M // blocking
        pat = torch.from_numpy(np.random.rand(R, R) < 0.5).to(dev)
        x = torch.randn(M, N, device=dev).to(dtype)
        x = (x.view(R, blocking, R, blocking) * pat.view(R, 1, R, 1)).reshape(M, N).contiguous()
        mask = kernels.block_mask(x, blocking)
        offsets, ri, ci = kernels.mask_to_topology(mask)
        nnz = ri.numel()
        data = kernels.gather_blocks(x, blocking, ri, ci, offsets)
        tag = f"8192^2 b={blocking} nnz={nnz}"
        add(f"block_mask {tag}", 2.0 * M * N, lambda: kernels.block_mask(x, blocking))
        add(f"gather_blocks {tag}", 4.0 * nnz * blocking * blocking, lambda: kernels.gather_blocks(x, blocking, ri, ci, offsets))
        add(f"to_dense {tag}", 2.0 * M * N + 2.0 * nnz * blocking * blocking,
            lambda: kernels.to_dense(data, offsets, ci, R, R, blocking))
        if blocking == 128:
            add(f"to_sparse (all phases incl. transpose and the count read-back) {tag}",
                2.0 * M * N + 4.0 * nnz * blocking * blocking, lambda: stk.ops.to_sparse(x, blocking),
                "one host read-back inside")
        del x, data
    for nnz, Cb, R, note in ((16768, 1024, 262, "single-CTA path"), (236000, 7168, 2108, "multi-kernel path")):
        rows = (torch.arange(nnz, device=dev) // (nnz // R + 1)).to(torch.int16)
        cols = torch.randint(0, Cb, (nnz,), device=dev).to(torch.int16)
        add(f"transpose_meta nnz={nnz} Cb={Cb}", 4.0 * nnz + 6.0 * nnz + 4.0 * (Cb + 1),
            lambda: kernels.transpose_meta(rows, cols, Cb), note + "; latency-bound")
    R, nnz = 2108, 236096
    offsets = (torch.arange(R + 1, device=dev) * 112).to(torch.int32)
    out16 = torch.empty(nnz, dtype=torch.int16, device=dev)
    add(f"row_indices nnz={nnz}", 4.0 * (R + 1) + 2.0 * nnz,
        lambda: kernels.row_indices(None, None, offsets, None, out16), "latency-bound")
    for rows, hidden, E, cpb, tag in ((17024, 1024, 8, 32, "configs[1]"), (33536, 4096, 8, 112, "configs[4] / 8")):
        bin_rows = torch.full((E,), rows // 128 // E, dtype=torch.int32, device=dev)
        br = int(bin_rows.sum())
        add(f"dmoe_topology {tag} nnz={br * cpb}", (2 + 2 + 2 + 4) * br * cpb + 4.0 * (br + 1) + 4.0 * (E * cpb + 1),
            lambda: dmoe.topology_from_bins(bin_rows, br, cpb * 128, dtype, dev, materialize=False), "latency-bound")
        src = torch.randn(rows, hidden, device=dev).to(dtype)
        index = torch.randperm(rows, device=dev).to(torch.int32)
        add(f"gather_rows {tag} {rows}x{hidden}", 4.0 * rows * hidden, lambda: dmoe.gather_rows(src, index))
        add(f"scatter_rows {tag} {rows}x{hidden}", 4.0 * rows * hidden, lambda: dmoe.scatter_rows(src, index, rows))
        w = torch.rand(rows // 2, 2, device=dev)
        add(f"weighted_sum_rows top-2 {tag}", 2.0 * rows * hidden + 1.0 * rows * hidden,
            lambda: dmoe.weighted_sum_rows(src, index, w, rows // 2, 2))
    assert lib.device_status() == 0
    return results


def reference_triton(dev="cuda"):
    """The reference's own Triton kernels (stk/backend/triton_kernels.py:21-220, staged under
    oracle/_ref) on this GPU, on the configs[1] forward products and the configs[2] products, next to
    this library on the same operands."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "oracle"))
    import stage_reference
    ref = stage_reference.import_reference()
    if ref is None:
        print("reference not staged (run python oracle/stage_reference.py where the reference is present)")
        return []
    lines = []
    for tag, (T, h, f, E, dtype, zipf) in (("configs[1]", (16384, 1024, 4096, 8, torch.float16, False)),
                                          ("configs[2]", (32768, 2048, 8192, 16, torch.bfloat16, True))):
        g = torch.Generator().manual_seed(0)
        p = (torch.arange(E) + 1.0) ** -1.2 if zipf else torch.ones(E)
        ids = torch.multinomial(p / p.sum(), T, replacement=True, generator=g).to(dev)
        _, padded, _, total = dmoe.route_top1(ids, E)
        topo = dmoe.block_diagonal_topology(padded, f, dtype, dev)
        nnz = topo.data.shape[0]
        rand = lambda *shape: torch.empty(*shape, dtype=dtype, device=dev).normal_(0, 0.02)
        x, w1, w2, dy = rand(total, h), rand(h, E * f), rand(E * f, h), rand(total, h)
        mine = stk.ops.sdd(x, w1, topo)
        rtopo = ref.Matrix(topo.size(), mine.data, topo.row_indices, topo.column_indices, topo.offsets,
                           topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
        flops = 2.0 * nnz * 128 * 128 * h
        specs = [("sdd x@w1", lambda: stk.ops.sdd(x, w1, topo), lambda: ref.ops.sdd(x, w1, rtopo)),
                 ("dsd h@w2", lambda: stk.ops.dsd(mine, w2), lambda: ref.ops.dsd(rtopo, w2)),
                 ("dsd h^T@dy", lambda: stk.ops.dsd(mine.t(), dy), lambda: ref.ops.dsd(rtopo.t(), dy)),
                 ("dds x^T@dh", lambda: stk.ops.dds(x.t(), mine), lambda: ref.ops.dds(x.t(), rtopo))]
        with torch.no_grad():
            for name, fn, rfn in specs:
                got, want = fn(), rfn()
                got = got.data if isinstance(got, stk.Matrix) else got
                want = want.data if hasattr(want, "row_indices") else want
                err = (got.float() - want.float()).abs().max().item() / max(want.float().pow(2).mean().sqrt().item(), 1e-30)
                ms = time_interleaved({"stk_b200": fn, "reference_triton": rfn})
                lines.append({"config": tag, "product": name, "stk_b200_tflops": round(flops / ms["stk_b200"] / 1e9, 1),
                              "reference_triton_tflops": round(flops / ms["reference_triton"] / 1e9, 1),
                              "speedup": round(ms["reference_triton"] / ms["stk_b200"], 2),
                              "max_abs_diff_over_rms": round(err, 5)})
                print(lines[-1], flush=True)
    return lines


def single(density=0.25, dev="cuda"):
    """A few launches of s @ b, a @ s and sdd on one random topology, kernel chosen by
    STK_B200_PAIR_MODE: the small case for a profiler capture."""
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
    """Forward + backward of the experts' MLP on the configs[1] shape (T=16384, h=1024, f=4096, E=8, fp16):
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


def products_fp8(dev="cuda", experts=8, rows_per_expert=4096, hidden=4096, ffn=14336):
    """The forward products of one GPU's share of the dMoE-XL layer (BASELINE configs[4] / 8) with
    float8_e4m3fn operands against the same products in bfloat16 and against cuBLASLt's float8 GEMM
    (torch._scaled_mm, unit scales) of the same useful FLOPs.  The weights are stored as in bench.py:
    w1 [E*f, h] (K contiguous), w2 [E*f, h] row-major (N contiguous), in both formats."""
    from stk_b200 import dmoe
    f8 = torch.float8_e4m3fn
    rows = experts * rows_per_expert
    bins = torch.full((experts,), rows_per_expert // 128, dtype=torch.int32, device=dev)
    topo = dmoe.topology_from_bins(bins, rows // 128, ffn, torch.bfloat16, dev, materialize=False)
    x = torch.randn(rows, hidden, device=dev, dtype=torch.bfloat16)
    w1 = torch.randn(experts * ffn, hidden, device=dev, dtype=torch.bfloat16) * 0.02      # [E*f, h]
    w2 = torch.randn(experts * ffn, hidden, device=dev, dtype=torch.bfloat16) * 0.02      # [E*f, h]
    x8, w18, w28 = x.to(f8), w1.to(f8), w2.to(f8)
    act = stk.ops.sdd(x, w1.t(), topo)
    act8 = stk.Matrix(topo.size(), act.data.to(f8), topo.row_indices, topo.column_indices, topo.offsets,
                      topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
    y = torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16)
    one = torch.ones((), device=dev)
    wa8, wb8 = w18[:ffn], w28[:ffn].t().contiguous()                 # one expert's weights, K contiguous, for the dense twins
    a28 = torch.randn(rows, ffn, device=dev, dtype=torch.bfloat16).to(f8)
    flops = 2.0 * rows * ffn * hidden
    out = []
    for name, fn16, fn8, twin in (
            ("sdd x@w1", lambda: stk.ops.sdd(x, w1.t(), topo), lambda: stk.ops.sdd(x8, w18.t(), topo),
             lambda: torch._scaled_mm(x8, wa8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)),
            ("dsd h@w2", lambda: stk.ops.dsd(act, w2, out=y), lambda: stk.ops.dsd(act8, w28, out=y),
             lambda: torch._scaled_mm(a28, wb8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16))):
        ms = time_interleaved({"bf16": fn16, "fp8": fn8, "cublaslt_fp8": twin}, rounds=5, iters=4)
        out.append({"product": name, "bf16_tflops": round(flops / ms["bf16"] / 1e9, 1),
                    "fp8_tflops": round(flops / ms["fp8"] / 1e9, 1),
                    "cublaslt_fp8_tflops": round(flops / ms["cublaslt_fp8"] / 1e9, 1),
                    "fp8_vs_cublaslt": round(ms["cublaslt_fp8"] / ms["fp8"], 3), "fp8_us": round(ms["fp8"] * 1e3, 1)})
    return out


def products_small_blocks(dev="cuda", size=8192, density=0.25):
    """Products with 64- and 32-blocks (run inside their containing 128-blocks) beside the same products with
    128-blocks at the same density; useful TFLOP/s count the small blocks' own elements only.  Two 64-block
    topologies: `clustered` = every kept 128-block is full of small blocks (no MMA work wasted), `scattered`
    = small blocks kept independently (at density d a 128-block is kept with probability 1 - (1-d)^4 and is
    a quarter to fully used).  Also the copy kernel alone, in GB/s of the bytes it reads and writes."""
    from stk_b200.ops import small_blocks
    dtype = torch.bfloat16
    out = []
    b = torch.randn(size, size, device=dev).to(dtype)
    a = torch.randn(size, size, device=dev).to(dtype)
    for blocking, kind in ((128, "as is"), (64, "clustered"), (64, "scattered"), (32, "scattered")):
        np.random.seed(0)
        if kind == "clustered":
            big = stk.random.mask(size, size, 1 - density, 128)
            keep = stk.ops.to_dense(big.to(dev)).to(dtype)
            topo = stk.ops.to_sparse(keep, blocking)
        else:
            topo = stk.random.mask(size, size, 1 - density, blocking).to(dev)
        nnz = topo.data.shape[0]
        s = stk.Matrix(topo.size(), torch.randn(nnz, blocking, blocking, device=dev).to(dtype), topo.row_indices,
                       topo.column_indices, topo.offsets, topo.column_indices_t, topo.offsets_t, topo.block_offsets_t)
        flops = 2.0 * nnz * blocking * blocking * size
        ms = time_interleaved({"dsd": lambda: stk.ops.dsd(s, b), "sdd": lambda: stk.ops.sdd(a, b, s)}, rounds=3, iters=3)
        row = {"blocking": blocking, "topology": kind, "blocks": nnz,
               "dsd_us": round(ms["dsd"] * 1e3, 1), "dsd_tflops": round(flops / ms["dsd"] / 1e9, 1),
               "sdd_us": round(ms["sdd"] * 1e3, 1), "sdd_tflops": round(flops / ms["sdd"] / 1e9, 1),
               "containing_128_blocks": nnz, "copy_us": None, "copy_gbs": None}
        if blocking != 128:
            coarse = small_blocks.coarse_topology(s)
            big_vals = torch.zeros((coarse.blocks, 128, 128), dtype=dtype, device=dev)
            copy_ms = _time_ms(lambda: kernels.regroup_blocks(s.data, big_vals, coarse.slot, True), iters=10, warm=3)
            row.update(containing_128_blocks=coarse.blocks, copy_us=round(copy_ms * 1e3, 1),
                       copy_gbs=round(2.0 * s.data.numel() * 2 / copy_ms / 1e6, 1))
        out.append(row)
    return out


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "c2"
    if which == "train":
        train_step()
    elif which == "ref":
        reference_triton()
    else:
        with torch.no_grad():
            if which == "single":
                single(float(sys.argv[2]) if len(sys.argv) > 2 else 0.25)
            elif which == "meta":
                for r in meta_kernels(peak_gbs=6549.4):
                    print(f"| {r['kernel']} | {r['algorithmic_mb']} | {r['us']} | {r['gbs']} | {r['frac']} | {r['note']} |", flush=True)
            elif which == "fp8":
                print("| product | bf16 TFLOP/s | fp8 TFLOP/s | fp8 us | cuBLASLt fp8 TFLOP/s | fp8 / cuBLASLt |\n|---|---|---|---|---|---|")
                for r in products_fp8():
                    print(f"| {r['product']} | {r['bf16_tflops']} | {r['fp8_tflops']} | {r['fp8_us']} | {r['cublaslt_fp8_tflops']} | {r['fp8_vs_cublaslt']} |", flush=True)
            elif which == "small":
                print("| blocking | topology | blocks | containing 128-blocks | dsd us | dsd useful TFLOP/s | sdd us | sdd useful TFLOP/s | copy us | copy GB/s |\n|---|---|---|---|---|---|---|---|---|---|")
                for r in products_small_blocks():
                    print(f"| {r['blocking']} | {r['topology']} | {r['blocks']} | {r['containing_128_blocks']} | {r['dsd_us']} | {r['dsd_tflops']} | {r['sdd_us']} | {r['sdd_tflops']} | {r['copy_us']} | {r['copy_gbs']} |", flush=True)
            elif which == "c2":
                info, lines = products_c2(all_modes=True)
                _print_table(f"dMoE fwd+bwd products, T=32768 h=2048 f=8192 E=16 bf16; {info}", lines)
            elif which == "c3":
                for density, res in products_c3(all_modes=True).items():
                    _print_table(f"\nrandom topology 8192^2, density {density}: {res['blocks']} blocks", res["lines"])
