"""Benchmark of the block-sparse matmul hot path: one forward pass of a sharded dMoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--shrink S] [--timeline]

Workload (BASELINE.json configs[4], bf16, 128x128 blocks): T = 131072 tokens, hidden 4096, ffn 14336 per
expert, E = 64 experts, top-2 routing from the softmax of N(0,1) logits, every expert's bin padded to
a multiple of 128 rows; per token  out = sum_j p_j * (GeLU(x @ w1[e_j]) @ w2[e_j]).
N = 1: the whole layer on one GPU.  N > 1 (launched with torch.distributed.run, one rank per GPU):
rank g holds T/N of the tokens and E/N of the experts (their weights never move); token rows travel
to their experts' GPUs and the results back over NVLink (strong scaling: the total work is fixed).

The metric is nnz-block TFLOP/s: the useful FLOPs of the two block-sparse products,
2 * nnz * 128 * 128 * hidden each, summed over all ranks, divided by the device time of the whole
step (routing, token movement / exchange, topology build, sdd with fused GeLU, dsd, weighted combine).

`--shrink S` divides tokens and experts by S (S = 8: the per-GPU problem of an 8-GPU run on one GPU; a
small case for profilers).  `--impl reference` times the reference's CPU formulation of the same step
(to_dense + torch.mm + mask) on the host cores, on a bounded sample of the workload.
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

T_TOKENS, HIDDEN, FFN, EXPERTS, TOP_K = 131072, 4096, 14336, 64, 2
DTYPE = torch.bfloat16
TOKEN_BLOCK = 16384          # tokens are generated in blocks of this size, each from its own seed
METRIC = "nnz_block_tflops_dmoe_xl_fwd_sdd_dsd"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, recorded from an ncu capture of
# `python bench.py --shrink 8 --kernels-only` (see profiles/); scaled by the blocks of the launch.
NCU_DRAM_BYTES_PER_BLOCK = 155033   # (5.14 GB sdd+gelu + 3.89 GB dsd) / 2 launches / 29120 blocks


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), float(d["hbm_gbs"]), "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


_SAMPLER_CODE = r"""
import json, signal, sys, time
import pynvml
index, period = int(sys.argv[1]), float(sys.argv[2])
pynvml.nvmlInit()
handle = pynvml.nvmlDeviceGetHandleByIndex(index)
smax = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
stop = []
signal.signal(signal.SIGTERM, lambda *a: stop.append(1))
print("ready", flush=True)
sm, mask = [], 0
while not stop:
    sm.append(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
    mask |= pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
    time.sleep(period)
print(json.dumps({"sm": sm, "mask": mask, "smax": smax}), flush=True)
"""


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while the timed region runs.

    The polling runs in a child process: a thread in this process competes for the interpreter lock
    with the launch loop."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, index, period_s=None):
        if period_s is None:
            period_s = float(os.environ.get("STK_BENCH_CLOCK_PERIOD_MS", "5")) / 1e3
        self.index, self.period = index, period_s
        self.proc, self.error = None, None

    def start(self):
        import subprocess
        # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES if it lists indices
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = self.index
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                phys = int(ids[self.index])
        try:
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_CODE, str(phys), str(self.period)],
                                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            if self.proc.stdout.readline().strip() != "ready":
                raise RuntimeError(self.proc.stderr.read()[-300:])
        except Exception as exc:  # NVML missing: report, do not fail the benchmark
            self.error = repr(exc)
            if self.proc is not None:
                self.proc.kill()
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + str(self.error)]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
            data = json.loads(out.strip().splitlines()[-1])
        except Exception as exc:
            self.proc.kill()
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampler failed: " + repr(exc)]}
        reasons = [name for name, bit in self.REASONS if data["mask"] & bit]
        return {"sm_mhz": statistics.median(data["sm"]) if data["sm"] else None, "sm_max_mhz": data["smax"],
                "reasons": reasons, "samples": len(data["sm"])}


# ------------------------------------------------------------------------------ synthetic inputs
# Everything is a function of global indices (expert id, token block), never of the rank count, so
# that the layer computes the same thing on 1, 2, 4 or 8 GPUs.
def expert_weights(e, dev):
    """(w1_e [hidden, ffn], w2_e [ffn, hidden]) ~ N(0, 0.02), from the expert's own seed."""
    g = torch.Generator(device=dev).manual_seed(1000 + e)
    w1 = torch.empty(HIDDEN, FFN, dtype=DTYPE, device=dev).normal_(0, 0.02, generator=g)
    w2 = torch.empty(FFN, HIDDEN, dtype=DTYPE, device=dev).normal_(0, 0.02, generator=g)
    return w1, w2


def local_weights(first_expert, n_experts, dev):
    """(w1 [hidden, n*ffn], w2 [n*ffn, hidden]) of a rank's experts.  w1 is STORED as [n*ffn, hidden]
    (one row per ffn unit, like a linear layer's weight) and handed to sdd as the transposed view: a
    64-row operand tile of a row-major [hidden, 64*14336] matrix touches 64 different 2 MB pages
    (1.8 MB between rows), and at that size the products were measured 20 % slower for it."""
    w1_store = torch.empty(n_experts * FFN, HIDDEN, dtype=DTYPE, device=dev)
    w2 = torch.empty(n_experts * FFN, HIDDEN, dtype=DTYPE, device=dev)
    for le in range(n_experts):
        a, b = expert_weights(first_expert + le, dev)
        w1_store[le * FFN:(le + 1) * FFN] = a.t()
        w2[le * FFN:(le + 1) * FFN] = b
    return w1_store.t(), w2


def token_rows(first_token, n_tokens, dev):
    """Tokens [first_token, first_token + n_tokens) ~ N(0, 0.02), generated block by block."""
    assert first_token % TOKEN_BLOCK == 0 and n_tokens % TOKEN_BLOCK == 0
    x = torch.empty(n_tokens, HIDDEN, dtype=DTYPE, device=dev)
    for i in range(n_tokens // TOKEN_BLOCK):
        g = torch.Generator(device=dev).manual_seed(7 + first_token // TOKEN_BLOCK + i)
        x[i * TOKEN_BLOCK:(i + 1) * TOKEN_BLOCK].normal_(0, 0.02, generator=g)
    return x


def routing(tokens, experts):
    """Top-2 of softmax(N(0,1) logits), seed 0: (expert ids int32 [T, 2], probabilities float32 [T, 2])."""
    g = torch.Generator().manual_seed(0)
    probs = torch.softmax(torch.randn(tokens, experts, generator=g), dim=1)
    p, ids = torch.topk(probs, TOP_K, dim=1)
    return ids.to(torch.int32), p.contiguous()


class Layer:
    """The dMoE layer of one rank: its experts' weights and the step that runs on device tensors."""

    def __init__(self, rank, world, dev, tokens, experts, chunks):
        import stk_b200 as stk
        from stk_b200 import dmoe
        self.stk, self.dmoe = stk, dmoe
        self.rank, self.world, self.dev = rank, world, dev
        self.tokens_total, self.experts_total = tokens, experts
        self.tokens, self.local = tokens // world, experts // world
        self.w1, self.w2 = local_weights(rank * self.local, self.local, dev)
        self.exchange = None
        if world > 1:
            self.exchange = dmoe.PeerExchange(experts, self.tokens, HIDDEN, HIDDEN, DTYPE, dev, top_k=TOP_K,
                                              chunks=chunks)
        self.last_topology = None

    def topology(self, bin_rows, block_rows):
        """The block-diagonal topology of rows in padded expert order, with the pair kernels' work-item
        table computed (it hangs on the topology's index tensor; both products use it)."""
        from stk_b200.backend import kernels
        topo = self.dmoe.topology_from_bins(bin_rows, block_rows, FFN, DTYPE, self.dev, materialize=False)
        kernels.pair_plan(topo.offsets, topo.column_indices)
        return topo

    def experts_mlp(self, x_rows, bin_rows, block_rows, first_local_expert, out=None, topo=None):
        """sdd -> GeLU -> dsd on rows in padded expert order; the GeLU runs in the SDD kernel's epilogue
        (stk.ops.sdd_gelu), so this is two kernel launches (plus the two small kernels of `topology`)."""
        n = bin_rows.numel()
        if topo is None:
            topo = self.topology(bin_rows, block_rows)
        c0, c1 = first_local_expert * FFN, (first_local_expert + n) * FFN
        self.last_topology = topo
        return self.stk.ops.dsd(self.stk.ops.sdd_gelu(x_rows, self.w1[:, c0:c1], topo), self.w2[c0:c1], out=out)

    def step(self, x, ids, probs):
        """One forward pass on this rank's tokens: [tokens, hidden] -> [tokens, hidden]."""
        dmoe = self.dmoe
        if self.exchange is None:
            index, position, padded, bin_rows, total = dmoe.route_topk(ids, self.experts_total)
            xp = dmoe.permute_tokens(x, index, total, top_k=TOP_K)
            y = self.experts_mlp(xp, bin_rows, total // 128, 0)
            return dmoe.combine_tokens(y, position, probs, x.shape[0], TOP_K)
        per, chunks = self.local, self.exchange.chunks

        def run_chunk(c, rows, bin_rows, block_rows, out, topo):
            self.experts_mlp(rows, bin_rows, block_rows, -(-c * per // chunks), out=out, topo=topo)
        return self.exchange.forward(x, ids, probs, run_chunk,
                                     prepare_fn=lambda c, bin_rows, block_rows: self.topology(bin_rows, block_rows))


def reference_rows(layer, x, ids, probs, sample):
    """out[t] for the sampled local tokens from first principles, in fp32 with the one intermediate
    rounding the pipeline has (the hidden activations are stored in bf16): sum_j p_j * GeLU(x W1_e) W2_e,
    the experts' weights regenerated from their seeds (they may live on another rank)."""
    dev = layer.dev
    xs = x[sample].float()
    out = torch.zeros(len(sample), HIDDEN, dtype=torch.float32, device=dev)
    ids_s, p_s = ids[sample].long(), probs[sample].float()
    for e in torch.unique(ids_s).tolist():
        w1, w2 = expert_weights(e, dev)
        hit = (ids_s == e)
        rows = torch.nonzero(hit.any(1)).view(-1)
        act = torch.nn.functional.gelu(xs[rows] @ w1.float()).to(DTYPE).float()
        y = (act @ w2.float()).to(DTYPE).float()
        weight = (p_s[rows] * hit[rows].float()).sum(1, keepdim=True)
        out[rows] += weight * y
    return out


def parity_check(layer, x, ids, probs, n_sample=48):
    """Outside the timed region: the layer's output for a sample of this rank's tokens against
    reference_rows, |out - ref| <= 3 * (1e-2 * RMS(ref) + 1e-2 * |ref|) (three 16-bit roundings lie
    between them: activations, expert output, combined output).  Returns the worst excess / RMS."""
    with torch.no_grad():
        out = layer.step(x, ids, probs)
        g = torch.Generator().manual_seed(11 + layer.rank)
        sample = torch.randperm(x.shape[0], generator=g)[:n_sample].to(layer.dev)
        ref = reference_rows(layer, x, ids, probs, sample)
        got = out[sample].float()
        rms = ref.pow(2).mean().sqrt().item()
        excess = (got - ref).abs() - 3 * (1e-2 * rms + 1e-2 * ref.abs())
        finite = bool(torch.isfinite(got).all())
        return (excess.max().item() / max(rms, 1e-30)) if finite else float("inf")


def timed(fn, steps, min_seconds=0.25, max_repeats=25, head_start=True, agree=None):
    """Median over R repeats of the CUDA-event time of `steps` back-to-back calls; R is chosen after the
    first repeat so that the repeats together last min_seconds.  `agree(ms)` returns the value all
    ranks settle on (the maximum), so that every rank runs the same number of steps.  Returns
    (ms per step, R)."""
    def once():
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        if head_start:
            torch.cuda._sleep(5_000_000)   # lets the host run ahead so that launch latency is not timed
        ev[0].record()
        for _ in range(steps):
            fn()
        ev[1].record()
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]) / steps
    times = [once()]
    first = agree(times[0]) if agree is not None else times[0]
    repeats = int(min(max_repeats, max(1, -(-min_seconds * 1e3 // max(first * steps, 1e-6)))))
    for _ in range(repeats - 1):
        times.append(once())
    return statistics.median(times), repeats


def launches_per_step(world, chunks):
    """Kernels of libstk_b200.so that one step of rank 0 launches (every one of them is this
    library's: no torch or vendor-library kernel runs inside a step)."""
    sort = 4                                   # slots by expert: count, group prefix, scan, scatter
    per_chunk = 4                              # topology, work-item table, sdd + gelu, dsd
    if world == 1:
        return sort + 1 + 1 + 1 + per_chunk + 1    # + count read-back, bin index, row gather, weighted sum
    # share counts, 2 + chunks + 1 barriers, plan, totals read-back, padding, pushes, returns, weighted sum
    return sort + 1 + (3 + chunks) + 1 + 1 + 1 + chunks + chunks * (per_chunk + 1) + 1


def run_ours(args):
    import stk_b200 as stk
    from stk_b200 import dmoe
    from stk_b200.backend import lib
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with "
                         "python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    torch.cuda.set_device(dev)
    cores_near_gpu = dmoe.bind_host_to_gpu_node(dev) if os.environ.get("STK_B200_BIND_HOST", "1") == "1" else 0
    if distributed:
        dist.init_process_group("nccl", device_id=dev)
    lib.load()
    tokens_total, experts_total = T_TOKENS // args.shrink, EXPERTS // args.shrink
    if experts_total % world or tokens_total % (world * TOKEN_BLOCK):
        raise SystemExit(f"{experts_total} experts / {tokens_total} tokens do not divide over {world} ranks")
    # expert chunks of the overlapped exchange: at least four experts per chunk (shorter products lose
    # more to their last, partly filled round of work items than the overlap gains), at most four chunks
    local_experts = experts_total // world
    chunks = int(os.environ.get("STK_B200_EP_CHUNKS", str(min(4, max(1, local_experts // 4)))))
    layer = Layer(rank, world, dev, tokens_total, experts_total, min(chunks, local_experts))
    tokens = layer.tokens
    ids_all, probs_all = routing(tokens_total, experts_total)
    sl = slice(rank * tokens, (rank + 1) * tokens)
    x_dev = token_rows(rank * tokens, tokens, dev)
    ids_dev, probs_dev = ids_all[sl].to(dev), probs_all[sl].to(dev)
    x_host = x_dev.cpu().pin_memory()
    ids_host, probs_host = ids_all[sl].contiguous().pin_memory(), probs_all[sl].contiguous().pin_memory()
    # this rank's share of the useful work: the padded rows of its experts
    counts = torch.bincount(ids_all.reshape(-1).long(), minlength=experts_total)
    padded = ((counts + 127) // 128) * 128
    rows_local = int(padded[rank * layer.local:(rank + 1) * layer.local].sum())
    nnz_local = rows_local // 128 * (FFN // 128)
    nnz_total = int(padded.sum()) // 128 * (FFN // 128)
    flops_product_local = 2.0 * nnz_local * 128 * 128 * HIDDEN
    flops_step_total = 2 * 2.0 * nnz_total * 128 * 128 * HIDDEN

    with torch.no_grad():
        # ---------------- parity of the layer, once per run, on every rank
        excess = parity_check(layer, x_dev, ids_dev, probs_dev)

        # ---------------- device-resident leg: tokens and routing already in HBM
        step = lambda: layer.step(x_dev, ids_dev, probs_dev)
        for _ in range(args.warmup):
            step()
        if args.timeline:
            print_timeline(step, rank, distributed)
            if distributed:
                dist.destroy_process_group()
            return
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()      # before the barrier: the other ranks must not time its start-up
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        def agree(ms):
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()
        ms_step, repeats = timed(step, args.steps, head_start=not distributed, agree=agree if distributed else None)
        if distributed:
            dist.barrier()
        clocks = sampler.stop() if rank == 0 else None

        # ---------------- the two products alone (rows already in expert order), per launch
        if distributed:
            xq, bins, st = layer.exchange.dispatch(x_dev, ids_dev)
            block_rows = st["block_rows"]
        else:
            index, position, _, bins, total = dmoe.route_topk(ids_dev, experts_total)
            xq = dmoe.permute_tokens(x_dev, index, total, top_k=TOP_K)
            block_rows = total // 128
        topo = dmoe.topology_from_bins(bins, block_rows, FFN, DTYPE, dev, materialize=False)
        k_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
        act = stk.ops.sdd_gelu(xq, layer.w1, topo)
        y = stk.ops.dsd(act, layer.w2)
        torch.cuda.synchronize()
        torch.cuda._sleep(5_000_000)
        for i in range(args.steps):
            k_ev[i][0].record()
            act = stk.ops.sdd_gelu(xq, layer.w1, topo)
            k_ev[i][1].record()
            stk.ops.dsd(act, layer.w2, out=y)
            k_ev[i][2].record()
        torch.cuda.synchronize()
        ms_sdd = statistics.median(e[0].elapsed_time(e[1]) for e in k_ev)
        ms_dsd = statistics.median(e[1].elapsed_time(e[2]) for e in k_ev)
        # launch path alone: host time per product call, nothing queued ahead of it
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(20):
            stk.ops.dsd(act, layer.w2, out=y)
        host_us = (time.perf_counter() - t0) / 20 * 1e6
        torch.cuda.synchronize()
        del act, y

        # cuBLAS on dense GEMMs with the same useful FLOPs: all padded rows against one expert's weights
        rows = block_rows * 128
        wa, wb = layer.w1[:, :FFN].contiguous(), layer.w2[:FFN].contiguous()
        a2 = torch.empty(rows, FFN, dtype=DTYPE, device=dev).normal_(0, 0.02)
        o1, o2 = torch.empty(rows, FFN, dtype=DTYPE, device=dev), torch.empty(rows, HIDDEN, dtype=DTYPE, device=dev)
        for _ in range(2):
            torch.matmul(xq, wa, out=o1), torch.matmul(a2, wb, out=o2)
        n_c = max(3, args.steps // 2)
        c_ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        torch.cuda._sleep(5_000_000)
        c_ev[0].record()
        for _ in range(n_c):
            torch.matmul(xq, wa, out=o1)
        c_ev[1].record()
        for _ in range(n_c):
            torch.matmul(a2, wb, out=o2)
        c_ev[2].record()
        torch.cuda.synchronize()
        ms_cublas_sdd = c_ev[0].elapsed_time(c_ev[1]) / n_c
        ms_cublas_dsd = c_ev[1].elapsed_time(c_ev[2]) / n_c
        del a2, o1, o2, wa, wb, xq

        # ---------------- end-to-end leg: host tokens and routing in, host result out, every step
        # Every step copies its own tokens and routing from pinned host memory and its own result
        # back; dmoe.HostPipeline lets the copies of neighbouring steps overlap the current one.
        e2e_steps = 0 if args.kernels_only else args.steps
        ms_e2e_total = 0.0
        if e2e_steps:
            pipe = dmoe.HostPipeline(lambda xd, idd, pd: layer.step(xd, idd, pd), dev)
            for _ in range(min(3, args.warmup)):
                pipe.submit(x_host, ids_host, probs_host)
            pipe.flush()
            torch.cuda.synchronize()
            if distributed:
                dist.barrier()
            e2e_ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            e2e_ev[0].record()
            for _ in range(e2e_steps):
                pipe.submit(x_host, ids_host, probs_host)
            pipe.flush()                       # the last result is in host memory when this returns
            e2e_ev[1].record()
            torch.cuda.synchronize()
            ms_e2e_total = e2e_ev[0].elapsed_time(e2e_ev[1])
        status = lib.device_status()

    # max over ranks of the timed regions and of the parity excess
    stats = torch.tensor([ms_step, ms_e2e_total, excess, float(status != 0)], dtype=torch.float64, device=dev)
    if distributed:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e_total, excess, any_status = (v.item() for v in stats)
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peak_tflops, peak_sustained, peak_gbs, peak_kind = measured_peaks()
    value = flops_step_total / (ms_step * 1e-3) / 1e12
    e2e_value = flops_step_total / (ms_e2e_total / args.steps * 1e-3) / 1e12 if e2e_steps else 0.0
    achieved = 2 * flops_product_local / ((ms_sdd + ms_dsd) * 1e-3) / 1e12
    # a launch of several milliseconds runs under the power cap: compare with the sustained peak
    long_launch = (ms_sdd + ms_dsd) / 2 > 2.0
    peak_used = peak_sustained if long_launch else peak_tflops
    shape = f"T={tokens_total} h={HIDDEN} f={FFN} E={experts_total} top-{TOP_K}"
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "sharded dMoE-XL layer forward, sdd->gelu->dsd (BASELINE.json configs[4]): " + shape
                               + (f" (shrunk by {args.shrink})" if args.shrink > 1 else ""),
                   "gelu": "fused into the SDD epilogue (fp32 accumulator, exact erf form)",
                   "weights": "w1 [h, E*f] stored as [E*f, h] (K-contiguous operand), w2 [E*f, h] row-major",
                   "step": "routing sort, token movement, topology build, sdd+gelu, dsd, weighted top-2 combine",
                   "tokens_per_gpu": tokens, "experts_per_gpu": layer.local, "blocking": 128,
                   "nnz_blocks_total": nnz_total, "nnz_blocks_rank0": nnz_local, "padded_rows_rank0": rows_local,
                   "parallelism": "1 GPU" if world == 1 else (
                       f"expert-parallel x{world}: token rows pushed to the experts' GPUs and results pushed back over "
                       f"NVLink peer memory by the library's kernels, {layer.exchange.chunks} expert chunks overlapped "
                       "with the products"),
                   "repeats": repeats, "timing": "median over repeats of CUDA-event time of `steps` steps",
                   "l2": "no flush: one step streams several GB (weights, activations) through the 126 MB L2"},
        "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": x_host.numel() * 2 + ids_host.numel() * 4 + probs_host.numel() * 4,
                "d2h_bytes_per_step": tokens * HIDDEN * 2,
                "includes": "per step and rank: H2D tokens + routing, the whole device step, D2H result",
                "overlap": "dmoe.HostPipeline: H2D of step i+1 and D2H of step i-1 run on their own streams "
                           "while step i computes",
                "host_cores_near_gpu": cores_near_gpu},
        "gpu_launches": launches_per_step(world, 1 if world == 1 else layer.exchange.chunks) * args.steps * repeats,
        "gpu_launches_per_step": launches_per_step(world, 1 if world == 1 else layer.exchange.chunks),
        "clocks": clocks,
        "parity": {"checked": True, "ok": bool(excess <= 0.0), "max_excess": round(excess, 5),
                   "what": "48 sampled tokens per rank vs fp32 per-expert MLP from regenerated weights; "
                           "excess = (|out-ref| - 3*(1e-2*RMS + 1e-2*|ref|)) / RMS, max over ranks, <= 0 passes"},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": peak_used,
                     "unit": "TFLOP/s", "frac": round(achieved / peak_used, 4),
                     "traffic": None if NCU_DRAM_BYTES_PER_BLOCK is None else NCU_DRAM_BYTES_PER_BLOCK * nnz_local,
                     "traffic_unit": "DRAM bytes per launch (mean of the two), scaled by blocks from a recorded ncu capture of the 1/8 case",
                     "algorithmic_flops_per_launch": flops_product_local,
                     "kernel": "bsmm_pair_kernel (sdd+gelu) and bsmm_wide_kernel (dsd): the two product launches of rank 0",
                     "peak_kind": peak_kind + (" bf16 sustained (launches of several ms run under the power cap)"
                                               if long_launch else " bf16 burst"),
                     "frac_of_burst_peak": round(achieved / peak_tflops, 4),
                     "nominal_frac": round(achieved / 2250.0, 4)},
        "kernels": {
            "sdd_ms": round(ms_sdd, 4), "sdd_tflops": round(flops_product_local / ms_sdd / 1e9, 1),
            "dsd_ms": round(ms_dsd, 4), "dsd_tflops": round(flops_product_local / ms_dsd / 1e9, 1),
            "products_only_ms": round(ms_sdd + ms_dsd, 4),
            "step_minus_products_ms": round(ms_step - ms_sdd - ms_dsd, 4),
            "cublas_same_flops_sdd_ms": round(ms_cublas_sdd, 4),
            "cublas_same_flops_sdd_tflops": round(flops_product_local / ms_cublas_sdd / 1e9, 1),
            "cublas_same_flops_dsd_ms": round(ms_cublas_dsd, 4),
            "cublas_same_flops_dsd_tflops": round(flops_product_local / ms_cublas_dsd / 1e9, 1),
            "sdd_vs_cublas": round(ms_cublas_sdd / ms_sdd, 4),
            "dsd_vs_cublas": round(ms_cublas_dsd / ms_dsd, 4),
            "host_us_per_call": round(host_us, 1)},
        "device_status": int(status) if not any_status else (int(status) or -10),
    }
    if world == 1 and not args.kernels_only:
        line.update(extra_sections(peak_gbs))
        line["cpu_baseline"] = cpu_baseline(repeats=2)
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def print_timeline(step, rank, distributed):
    """--timeline: start, end and duration (us, relative to the step's first kernel) of every kernel of
    one step on rank 0, both streams, from torch's profiler - where the exchange and the products
    overlap and where they wait for one another.  Not a timing run: the profiler slows the host."""
    import torch.distributed as dist
    from torch.profiler import profile, ProfilerActivity
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    if rank == 0:
        events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                        key=lambda e: e.time_range.start)
        last = events[2 * (len(events) // 3):]
        t0 = last[0].time_range.start
        for e in last:
            print(f"{e.time_range.start - t0:10.1f} {e.time_range.end - t0:10.1f} "
                  f"{e.time_range.end - e.time_range.start:9.1f} us  {e.name[:80]}", flush=True)
    if distributed:
        dist.barrier()


def extra_sections(peak_gbs):
    """The other benchmark configurations and the conversion kernels, one GPU: configs[1] (forward
    products, fp16), configs[2] (six forward + backward products), configs[3] (random sparsity sweep),
    each against cuBLAS of the same FLOPs; achieved GB/s of the metadata / conversion kernels; the
    float8 form of the dMoE forward products."""
    from stk_b200 import benchmarks
    torch.cuda.empty_cache()
    out = {}
    with torch.no_grad():
        out["c1"] = headline_c1()
        torch.cuda.empty_cache()
        info, lines = benchmarks.products_c2()
        out["c2"] = {"workload": "BASELINE.json configs[2]: T=32768 h=2048 f=8192 E=16 Zipf(1.2), bf16", **info,
                     "products": lines}
        torch.cuda.empty_cache()
        out["c3"] = {"workload": "BASELINE.json configs[3]: random block sparsity, 8192^3, bf16, seed 0",
                     "densities": benchmarks.products_c3()}
        torch.cuda.empty_cache()
        meta = benchmarks.meta_kernels(peak_gbs=peak_gbs)
        out["roofline_meta"] = {"bound": "hbm", "peak": peak_gbs, "unit": "GB/s",
                                "achieved": "algorithmic bytes / CUDA-event time per call", "kernels": meta}
        torch.cuda.empty_cache()
        out["fp8"] = {"workload": "the two forward products of BASELINE.json configs[4] / 8 (8 experts x 4096 rows, h=4096, "
                                  "f=14336) with float8_e4m3fn operands, bf16 output; against the same products in bf16 and "
                                  "against cuBLASLt's float8 GEMM of the same FLOPs (torch._scaled_mm), interleaved",
                      "products": None}
        try:
            out["fp8"]["products"] = benchmarks.products_fp8()
        except Exception as exc:      # the comparison leg uses a private torch entry point (torch._scaled_mm)
            out["fp8"]["error"] = f"{type(exc).__name__}: {exc}"[:300]
    return out


def headline_c1():
    """BASELINE.json configs[1] (fp16, T=16384, h=1024, f=4096, E=8, top-1): sdd+gelu and dsd against
    cuBLAS GEMMs of the same FLOPs."""
    import stk_b200 as stk
    from stk_b200 import benchmarks, dmoe
    dev, dtype, T, h, f, E = "cuda", torch.float16, 16384, 1024, 4096, 8
    g = torch.Generator().manual_seed(1234)
    ids = torch.multinomial(torch.full((E,), 1.0 / E), T, replacement=True, generator=g).to(dev).to(torch.int32)
    index, padded, bin_rows, total = dmoe.route_top1(ids, E)
    topo = dmoe.topology_from_bins(bin_rows, total // 128, f, dtype, dev)
    rand = lambda *shape: torch.empty(*shape, dtype=dtype, device=dev).normal_(0, 0.02)
    x, w1, w2 = rand(total, h), rand(h, E * f), rand(E * f, h)
    act = stk.ops.sdd_gelu(x, w1, topo)
    wa, wb, a2 = w1[:, :f].contiguous(), w2[:f].contiguous(), rand(total, f)
    flops = 2.0 * topo.data.shape[0] * 128 * 128 * h
    ms = benchmarks.time_interleaved({"sdd": lambda: stk.ops.sdd_gelu(x, w1, topo), "dsd": lambda: stk.ops.dsd(act, w2),
                                      "cublas_sdd": lambda: x @ wa, "cublas_dsd": lambda: a2 @ wb}, rounds=7, iters=8)
    return {"workload": "BASELINE.json configs[1]: T=16384 h=1024 f=4096 E=8 top-1, fp16", "blocks": topo.data.shape[0],
            "sdd_gelu_tflops": round(flops / ms["sdd"] / 1e9, 1), "dsd_tflops": round(flops / ms["dsd"] / 1e9, 1),
            "sdd_vs_cublas": round(ms["cublas_sdd"] / ms["sdd"], 3), "dsd_vs_cublas": round(ms["cublas_dsd"] / ms["dsd"], 3),
            "sdd_us": round(ms["sdd"] * 1e3, 1), "dsd_us": round(ms["dsd"] * 1e3, 1)}


# ------------------------------------------------------------------------------ CPU arms
def cpu_sample():
    """The bounded CPU sample of the workload: the padded rows of expert 0 (1/64 of the step) against
    that expert's weights.  Returns (reference module or None, topology, x, w1, w2, padded rows)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import stage_reference
    ref = stage_reference.import_reference()
    ids_all, _ = routing(T_TOKENS, EXPERTS)
    rows = int((ids_all == 0).sum())
    padded = (rows + 127) // 128 * 128
    g = torch.Generator().manual_seed(5)
    x = torch.zeros(padded, HIDDEN, dtype=DTYPE)
    x[:rows] = (torch.randn(rows, HIDDEN, generator=g) * 0.02).to(DTYPE)
    w1 = (torch.randn(HIDDEN, FFN, generator=g) * 0.02).to(DTYPE)
    w2 = (torch.randn(FFN, HIDDEN, generator=g) * 0.02).to(DTYPE)
    topo = ref.ops.to_sparse(torch.ones(padded, FFN, dtype=DTYPE), 128) if ref is not None else None
    return ref, topo, x, w1, w2, padded


def cpu_step(ref, topo, x, w1, w2, padded):
    """One expert's share of the step the way the reference computes it on the CPU
    (stk/ops/linear_ops_test.py:83-112): sdd as the dense product times to_dense(ones_like(topo)),
    GeLU on the sparse values, dsd as to_dense(sparse operand) @ dense."""
    if ref is not None:
        mask = ref.ops.to_dense(ref.ops.ones_like(topo))
        hidden = ref.ops.to_sparse(torch.mm(x, w1) * mask, 128)
        act = ref.Matrix(hidden.size(), torch.nn.functional.gelu(hidden.data), hidden.row_indices,
                         hidden.column_indices, hidden.offsets, hidden.column_indices_t, hidden.offsets_t,
                         hidden.block_offsets_t)
        return torch.mm(ref.ops.to_dense(act), w2)
    from oracle import stk_oracle as oracle
    import numpy as np
    cpb = FFN // 128
    row_idx = np.repeat(np.arange(padded // 128), cpb).astype(np.int16)
    col_idx = np.tile(np.arange(cpb), padded // 128).astype(np.int16)
    ones = torch.ones((len(row_idx), 128, 128), dtype=DTYPE)
    hidden_dense = oracle.reference_cpu_path_sdd(x, w1, ones, row_idx, col_idx, (padded, FFN))
    return torch.mm(torch.nn.functional.gelu(hidden_dense), w2)


def cpu_baseline(repeats=2, warm=0):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = cpu_sample()
    ref, padded = sample[0], sample[-1]
    flops = 2 * (2.0 * padded * HIDDEN * FFN)
    for _ in range(warm):
        cpu_step(*sample)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_step(*sample)
        times.append(time.perf_counter() - t0)
    best = min(times)
    kind = "reference" if ref is not None else "port"
    how = ("the reference's own to_sparse / to_dense / ones_like (staged under oracle/_ref) + torch.mm"
           if ref is not None else "oracle port of the reference's dense formulation")
    return {"value": round(flops / best / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"padded rows of expert 0 of {EXPERTS} ({padded} rows x {FFN} columns, "
                      f"{padded // 128 * (FFN // 128)} blocks): {how}; best of {repeats}",
            "seconds": round(best, 3), "mean_seconds": round(sum(times) / len(times), 3), "rows": padded}


def run_reference(args):
    """The reference's CPU formulation, timed like a bench arm: W warm-up + K timed sample steps."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps, warmup = max(1, min(args.steps, 4)), max(0, min(args.warmup, 1))
    res = cpu_baseline(repeats=steps, warm=warmup)
    padded = res["rows"]
    flops = 2 * (2.0 * padded * HIDDEN * FFN)
    sec = res["mean_seconds"]
    value = round(flops / sec / 1e12, 4)
    res = dict(res, value=value)
    res["sample"] += f"; {steps} timed steps after {warmup} warm-up (requested {args.steps}/{args.warmup}, " \
                     "capped so the run ends within minutes), mean"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "sharded dMoE-XL layer forward, sdd->gelu->dsd (BASELINE.json configs[4]), CPU dense "
                               "formulation of the reference on a bounded sample (one expert's rows)"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--shrink", type=int, default=1, choices=(1, 2, 4, 8),
                    help="divide tokens and experts by this (8: the per-GPU problem of an 8-GPU run)")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernel timeline of one step on rank 0 instead of timing")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end, extra-configuration and CPU legs (short run for profilers)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
