"""Benchmark of the block-sparse matmul hot path: one dMoE forward step, sdd -> GeLU -> dsd.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: BASELINE.json configs[1] (dMoE forward, fp16, T=16384, h=1024, f=4096, E=8, top-1 routing,
128x128 blocks) on one GPU.  N > 1 (launched with torch.distributed.run, one rank per GPU): the
same per-GPU problem with expert parallelism - every rank owns 8 of the 8N experts and 16384 of
the tokens; tokens travel to their expert's GPU and back with NCCL all-to-all (weak scaling).

The metric is nnz-block TFLOP/s: 2 * nnz * 128 * 128 * D useful FLOPs of the two products divided by
the device time of the whole step (GeLU and, for N > 1, the exchanges included).

`--impl reference` times the reference's CPU formulation of the same step (to_dense + torch.mm +
mask, restated in oracle/stk_oracle.py) on the host cores, on a bounded sample of the workload.
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

T_TOKENS, HIDDEN, FFN, EXPERTS = 16384, 1024, 4096, 8   # per GPU
DTYPE = torch.float16
METRIC = "nnz_block_tflops_dmoe_fwd_sdd_dsd"
# dram__bytes_read.sum + dram__bytes_write.sum of the two bsmm_pair_kernel launches of one step, from the ncu
# capture summarised in profiles/bsmm_pair_kernel_dmoe_fwd.md (sdd+gelu 196.6 MB, dsd 239.4 MB), per launch.
NCU_DRAM_BYTES_PER_LAUNCH = (196.6e6 + 239.4e6) / 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


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
    with the launch loop, which slowed the host-bound multi-GPU step by a third."""

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


def expert_ids_for(rank, tokens, experts, device):
    g = torch.Generator().manual_seed(1234 + rank)
    return torch.multinomial(torch.full((experts,), 1.0 / experts), tokens, replacement=True,
                             generator=g).to(device)


def make_weights(rank, device):
    g = torch.Generator().manual_seed(99 + rank)
    w1 = (torch.randn(HIDDEN, EXPERTS * FFN, generator=g) * 0.02).to(DTYPE).to(device)
    w2 = (torch.randn(EXPERTS * FFN, HIDDEN, generator=g) * 0.02).to(DTYPE).to(device)
    return w1, w2


def make_tokens(rank):
    g = torch.Generator().manual_seed(7 + rank)
    return (torch.randn(T_TOKENS, HIDDEN, generator=g) * 0.02).to(DTYPE)


def expert_step(stk, x_padded, topo, w1, w2, out=None):
    """sdd -> GeLU -> dsd on tokens already in padded expert order; the GeLU runs in the SDD
    kernel's epilogue (stk.ops.sdd_gelu), so the step is two kernel launches.  `out`: where the
    second product is written (the exchange's result buffer on several GPUs)."""
    return stk.ops.dsd(stk.ops.sdd_gelu(x_padded, w1, topo), w2, out=out)


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
    if distributed:
        dist.init_process_group("nccl", device_id=dev)
    lib.load()

    w1, w2 = make_weights(rank, dev)
    x_host = make_tokens(rank).pin_memory()
    total_experts = EXPERTS * world
    ids = expert_ids_for(rank, T_TOKENS, total_experts, dev).to(torch.int32)
    ids_host = ids.cpu().pin_memory()
    exchange, exchange_kind = None, "none"
    if distributed:
        # Rows travel with this library's own kernels over peer memory; NCCL all-to-all only if torch's
        # symmetric memory cannot be set up here (or STK_B200_EXCHANGE=nccl asks for it).
        exchange_kind = os.environ.get("STK_B200_EXCHANGE", "peer")
        if exchange_kind == "peer":
            try:
                exchange = dmoe.PeerExchange(total_experts, T_TOKENS, HIDDEN, HIDDEN, DTYPE, dev)
            except Exception as exc:  # noqa: BLE001 - any failure of the symmetric allocation
                if rank == 0:
                    print(f"peer exchange unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
                exchange_kind = "nccl"
        if exchange is None:
            exchange = dmoe.ExpertParallelExchange(total_experts)

    def result_rows(state):
        return exchange.result_rows(state) if exchange_kind == "peer" else None

    def full_step(x_dev, ids_dev):
        """Routing bookkeeping + (exchange) + sdd -> GeLU -> dsd + (exchange back)."""
        if distributed:
            xp, bin_rows, state = exchange.dispatch(x_dev, ids_dev)
            topo = dmoe.topology_from_bins(bin_rows, state["block_rows"], FFN, DTYPE, dev)
            y = expert_step(stk, xp, topo, w1, w2, out=result_rows(state))
            return exchange.combine(y, state), topo
        index, padded, bin_rows, total = dmoe.route_top1(ids_dev, EXPERTS)
        topo = dmoe.topology_from_bins(bin_rows, total // 128, FFN, DTYPE, dev)
        y = expert_step(stk, dmoe.permute_tokens(x_dev, index, total), topo, w1, w2)
        return dmoe.unpermute_tokens(y, index, x_dev.shape[0]), topo

    with torch.no_grad():
        # ---------------- device-resident leg: inputs and topology already in HBM
        x_dev = x_host.to(dev)
        if distributed:
            xp, bin_rows, state = exchange.dispatch(x_dev, ids)
            block_rows = state["block_rows"]
        else:
            index, padded, bin_rows, total = dmoe.route_top1(ids, EXPERTS)
            xp = dmoe.permute_tokens(x_dev, index, total)
            block_rows = total // 128
        topo = dmoe.topology_from_bins(bin_rows, block_rows, FFN, DTYPE, dev)
        nnz = topo.data.shape[0]
        flops_sdd = 2.0 * nnz * 128 * 128 * HIDDEN
        flops_dsd = 2.0 * nnz * 128 * 128 * HIDDEN
        flops_step = flops_sdd + flops_dsd

        def resident_step():
            if distributed:
                xq, _, st = exchange.dispatch(x_dev, ids)
                y = expert_step(stk, xq, topo, w1, w2, out=result_rows(st))
                return exchange.combine(y, st)
            return expert_step(stk, xp, topo, w1, w2)

        for _ in range(args.warmup):
            resident_step()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()      # before the barrier: the other ranks must not time its start-up
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        if not distributed:
            torch.cuda._sleep(20_000_000)   # let the host run ahead so that launch latency is not timed
        ev[0].record()
        for _ in range(args.steps):
            resident_step()
        ev[1].record()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        ms_total = ev[0].elapsed_time(ev[1])
        clocks = sampler.stop() if rank == 0 else None

        # ---------------- per-kernel timing (same stream, events around each launch)
        k_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
        act = stk.ops.sdd_gelu(xp, w1, topo)
        torch.cuda.synchronize()
        torch.cuda._sleep(20_000_000)
        for i in range(args.steps):
            k_ev[i][0].record()
            act = stk.ops.sdd_gelu(xp, w1, topo)
            k_ev[i][1].record()
            stk.ops.dsd(act, w2)
            k_ev[i][2].record()
        torch.cuda.synchronize()
        ms_sdd = statistics.mean(e[0].elapsed_time(e[1]) for e in k_ev)
        ms_dsd = statistics.mean(e[1].elapsed_time(e[2]) for e in k_ev)

        # cuBLAS on dense GEMMs with the same useful FLOPs
        rows = topo.size()[0]
        a1, b1 = xp, w1[:, :FFN].contiguous()
        a2 = torch.empty(rows, FFN, dtype=DTYPE, device=dev).normal_(0, 0.02)
        b2 = w2[:FFN].contiguous()
        for _ in range(3):
            torch.matmul(a1, b1), torch.matmul(a2, b2)
        c_ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        torch.cuda._sleep(20_000_000)
        c_ev[0].record()
        for _ in range(args.steps):
            torch.matmul(a1, b1)
        c_ev[1].record()
        for _ in range(args.steps):
            torch.matmul(a2, b2)
        c_ev[2].record()
        torch.cuda.synchronize()
        ms_cublas_sdd = c_ev[0].elapsed_time(c_ev[1]) / args.steps
        ms_cublas_dsd = c_ev[1].elapsed_time(c_ev[2]) / args.steps

        # ---------------- end-to-end leg: host tokens and routing in, host result out, every step
        # Every step copies its own tokens and routing from pinned host memory and its own result
        # back; dmoe.HostPipeline lets the copies of neighbouring steps overlap the current one.
        e2e_steps = 0 if args.kernels_only else args.steps
        pipe = dmoe.HostPipeline(lambda xd, idd: full_step(xd, idd)[0], dev)
        for _ in range(0 if args.kernels_only else min(3, args.warmup)):
            pipe.submit(x_host, ids_host)
        pipe.flush()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        e2e_ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        e2e_ev[0].record()
        for _ in range(e2e_steps):
            pipe.submit(x_host, ids_host)
        pipe.flush()                       # the last result is in host memory when this returns
        e2e_ev[1].record()
        torch.cuda.synchronize()
        ms_e2e_total = e2e_ev[0].elapsed_time(e2e_ev[1])
        status = lib.device_status()

    # max over ranks of the timed regions; sum over ranks of the useful work
    stats = torch.tensor([ms_total, ms_e2e_total, flops_step], dtype=torch.float64, device=dev)
    if distributed:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_total, ms_e2e_total, flops_all = mx[0].item(), mx[1].item(), sm[2].item()
    else:
        flops_all = flops_step
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peak_tflops, peak_gbs, peak_kind = measured_peaks()
    ms_step = ms_total / args.steps
    value = flops_all / (ms_step * 1e-3) / 1e12
    e2e_value = flops_all / (ms_e2e_total / args.steps * 1e-3) / 1e12 if e2e_steps else 0.0
    achieved = (flops_sdd + flops_dsd) / ((ms_sdd + ms_dsd) * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": "dMoE forward sdd->gelu->dsd (BASELINE.json configs[1]) per GPU",
                   "gelu": "fused into the SDD epilogue (fp32 accumulator, exact erf form)",
                   "tokens_per_gpu": T_TOKENS, "hidden": HIDDEN, "ffn": FFN,
                   "experts_per_gpu": EXPERTS, "routing": "top-1 multinomial(uniform)",
                   "blocking": 128, "nnz_blocks_rank0": nnz, "padded_rows_rank0": rows,
                   "parallelism": "1 GPU" if world == 1 else (
                       f"expert-parallel x{world}, token rows pushed / pulled over NVLink peer memory by the library's kernels"
                       if exchange_kind == "peer" else f"expert-parallel x{world}, NCCL all-to-all"),
                   "l2": "no flush: operands + hidden + output of one step are ~335 MB > 126 MB L2"},
        "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": x_host.numel() * 2 + ids_host.numel() * 4,
                "d2h_bytes_per_step": T_TOKENS * HIDDEN * 2,
                "includes": "per step: H2D tokens+routing, routing/permute, topology build, (exchange), "
                            "sdd, gelu, dsd, un-permute, D2H result",
                "overlap": "dmoe.HostPipeline: H2D of step i+1 and D2H of step i-1 run on their own streams "
                           "while step i computes"},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": peak_tflops,
                     "unit": "TFLOP/s", "frac": round(achieved / peak_tflops, 4),
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "traffic_unit": "DRAM bytes per launch (ncu)",
                     "algorithmic_flops_per_launch": flops_sdd,
                     "kernel": "bsmm_pair_kernel (sdd+gelu and dsd launches)", "peak_kind": peak_kind + " bf16 burst",
                     "nominal_frac": round(achieved / 2250.0, 4)},
        "kernels": {
            "sdd_ms": round(ms_sdd, 4), "sdd_tflops": round(flops_sdd / ms_sdd / 1e9, 1),
            "dsd_ms": round(ms_dsd, 4), "dsd_tflops": round(flops_dsd / ms_dsd / 1e9, 1),
            "cublas_same_flops_sdd_ms": round(ms_cublas_sdd, 4),
            "cublas_same_flops_sdd_tflops": round(flops_sdd / ms_cublas_sdd / 1e9, 1),
            "cublas_same_flops_dsd_ms": round(ms_cublas_dsd, 4),
            "cublas_same_flops_dsd_tflops": round(flops_dsd / ms_cublas_dsd / 1e9, 1),
            "sdd_vs_cublas": round(ms_cublas_sdd / ms_sdd, 4),
            "dsd_vs_cublas": round(ms_cublas_dsd / ms_dsd, 4)},
        "device_status": status,
    }
    if world == 1 and not args.kernels_only:
        line["cpu_baseline"] = cpu_baseline(repeats=2)
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def cpu_sample():
    """The bounded CPU sample of the workload: the padded token rows of experts 0 and 1 (a quarter
    of the step), against all E*f columns, exactly as the reference's dense formulation would
    process them."""
    from oracle import stk_oracle as oracle
    import numpy as np
    ids = expert_ids_for(0, T_TOKENS, EXPERTS, "cpu")
    counts = torch.bincount(ids, minlength=EXPERTS)
    padded = ((counts + 127) // 128) * 128
    sample_experts = 2
    rows = int(padded[:sample_experts].sum())
    cpb = FFN // 128
    row_idx = np.repeat(np.arange(rows // 128), cpb).astype(np.int16)
    expert_of_row = np.repeat(np.arange(sample_experts), (padded[:sample_experts] // 128).numpy())
    col_idx = (expert_of_row[:, None] * cpb + np.arange(cpb)[None, :]).reshape(-1).astype(np.int16)
    w1, w2 = make_weights(0, "cpu")
    x = make_tokens(0)[:rows].contiguous()
    nnz = len(row_idx)
    return oracle, x, w1, w2, row_idx, col_idx, rows, nnz


def cpu_step(oracle, x, w1, w2, row_idx, col_idx, rows, nnz):
    """Reference CPU path of one step (stk/ops/linear_ops_test.py:83-112): dense product times the
    topology mask, GeLU, densified sparse operand times w2."""
    shape = (rows, EXPERTS * FFN)
    ones = torch.ones((nnz, 128, 128), dtype=DTYPE)
    hidden_dense = oracle.reference_cpu_path_sdd(x, w1, ones, row_idx, col_idx, shape)
    act = torch.nn.functional.gelu(hidden_dense)
    return torch.mm(act, w2)


def cpu_baseline(repeats=2):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = cpu_sample()
    nnz = sample[-1]
    flops = 2 * (2.0 * nnz * 128 * 128 * HIDDEN)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        cpu_step(*sample)
        best = min(best, time.perf_counter() - t0)
    return {"value": round(flops / best / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"padded rows of experts 0-1 of 8 ({sample[-2]} rows, {nnz} blocks), all "
                      f"{EXPERTS * FFN} columns: to_dense + torch.mm + mask, GeLU, torch.mm; "
                      f"best of {repeats}", "seconds": round(best, 3)}


def run_reference(args):
    """The reference's CPU formulation, timed like a bench arm: W warm-up + K timed sample steps."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = cpu_sample()
    nnz = sample[-1]
    flops = 2 * (2.0 * nnz * 128 * 128 * HIDDEN)
    steps, warmup = max(1, min(args.steps, 5)), max(0, min(args.warmup, 1))
    for _ in range(warmup):
        cpu_step(*sample)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(*sample)
    sec = (time.perf_counter() - t0) / steps
    value = round(flops / sec / 1e12, 4)
    desc = (f"padded rows of experts 0-1 of 8 ({sample[-2]} rows, {nnz} blocks) per step; "
            f"{steps} timed steps after {warmup} warm-up (requested {args.steps}/{args.warmup}, "
            "capped so the run ends within minutes)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": "dMoE forward sdd->gelu->dsd (BASELINE.json configs[1]), CPU dense "
                               "formulation of the reference on a bounded sample"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end and CPU legs (short run for profilers)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
