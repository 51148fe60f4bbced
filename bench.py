#!/usr/bin/env python
"""Benchmark of the matmul hot path: GEMM TFLOP/s at the large-square BFloat16 configuration
(C = A . B, 16384 x 16384 x 16384, row-major, fp32 accumulate, BFloat16 output).

  python bench.py --gpus N --steps K --warmup W            # this library (one rank per GPU)
  python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU algorithm

At N > 1 (launched by torch.distributed.run) the columns of B and C are sharded over the ranks,
no collective in the data path (strong scaling: the total work is fixed).  A "step" is one
matmul of the whole problem; `value` counts the algorithmic 2.M.N.K flops of all ranks over the
max-over-ranks device time.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, N, K, dtype, description)
    "bf16_16384": (16384, 16384, 16384, "bf16", "C = A.B 16384^3 BFloat16, uniform[-1,1), fp32 accumulate, BFloat16 out"),
    "bf16_8192": (8192, 8192, 8192, "bf16", "C = A.B 8192^3 BFloat16 (reduced size, not the headline)"),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # the clock under load: median of the upper half of the samples (idle samples drop out)
        sm.sort()
        upper = sm[len(sm) // 2:]
        return {"sm_mhz": upper[len(upper) // 2], "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
def cpu_inputs(N, K):
    """B of the workload as stored BFloat16 bits (seeded, uniform[-1,1)), made once per run."""
    import numpy as np
    from oracle import oracle
    rng = np.random.default_rng(0)
    b = np.empty((K, N), dtype=np.uint16)
    for r0 in range(0, K, 1024):                      # in slabs: keeps the float32 staging small
        blk = rng.random((min(1024, K - r0), N), dtype=np.float32) * 2.0 - 1.0
        b[r0:r0 + blk.shape[0]] = oracle.encode(blk, oracle.BF16)
    return b


def cpu_sample(M, N, K, b, threads=None, target_s=12.0):
    """Times the CPU restatement of the reference loop on a bounded row sample of the workload
    (same seeded value distribution), all host threads.  Returns (tflops, cores, description, seconds)."""
    import numpy as np
    from oracle import oracle
    if threads is None:
        # every core this process may run on (torchrun sets OMP_NUM_THREADS=1, which is not the machine)
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else oracle.lib().oracle_max_threads()
    rng = np.random.default_rng(1)
    probe_rows = threads * 8                      # one block of 8 rows per thread
    a = oracle.encode(rng.random((probe_rows, K), dtype=np.float32) * 2.0 - 1.0, oracle.BF16)
    t0 = time.perf_counter()
    oracle.matmul(a, b, oracle.BF16, threads=threads)
    probe = time.perf_counter() - t0
    rows = int(min(M, max(probe_rows, probe_rows * target_s / max(probe, 1e-6))))
    rows = max(probe_rows, rows // probe_rows * probe_rows)
    a = oracle.encode(rng.random((rows, K), dtype=np.float32) * 2.0 - 1.0, oracle.BF16)
    t0 = time.perf_counter()
    oracle.matmul(a, b, oracle.BF16, threads=threads)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * N * K / dt / 1e12
    desc = f"{rows} of {M} rows of A (all {N} columns, K={K}), k-outer loop order, {threads} OpenMP threads, {dt:.1f} s"
    return tflops, threads, desc, dt


def run_reference(args):
    """The reference arm: the reference's own CPU algorithm for this path (C restatement of
    cpu_matmul; the Swift original cannot be built without its toolchain) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M, N, K, dtype, desc = WORKLOADS[args.workload]
    vals, last = [], None
    b = cpu_inputs(N, K)
    for i in range(args.warmup + args.steps):
        last = cpu_sample(M, N, K, b, target_s=args.cpu_seconds / max(1, args.warmup + args.steps))
        if i >= args.warmup:
            vals.append(last)
    tflops = sum(v[0] for v in vals) / len(vals)
    ms = sum(v[3] for v in vals) / len(vals) * 1e3
    line = {
        "impl": "reference", "metric": "GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": desc, "M": M, "N": N, "K": K, "step": "bounded row sample of the workload on the host CPU"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": last[1], "kind": "port", "sample": last[2]},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def measure_e2e(args, srt, a, b, M, N, K, n_local, dev, world, barrier):
    """End to end: host buffers in, host result out, copies inside the timed region."""
    import torch
    import torch.distributed as dist
    tdt = a.dtype
    flops = 2.0 * M * N * K
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    ha = a.cpu().pin_memory()
    hb = b.contiguous().cpu().pin_memory()
    hc = torch.empty((M, n_local), dtype=tdt).pin_memory()
    srt.matmul_host(ha, hb, device=dev, out_host=hc)      # warm-up (allocator, pinned pages)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        srt.matmul_host(ha, hb, device=dev, out_host=hc)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    h2d = (ha.numel() + hb.numel()) * ha.element_size()
    d2h = hc.numel() * hc.element_size()
    bytes_t = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(bytes_t, op=dist.ReduceOp.SUM)
    return {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
            "h2d_bytes_per_step": int(bytes_t[0].item()), "d2h_bytes_per_step": int(bytes_t[1].item())}


def measure_gather(args, srt, a, b_full, M, N, K, dev, world, barrier):
    """Full C on every GPU, two ways, same sharding (N over the ranks), device-timed, max over ranks:
    fused  = srtMatmulAllGather: the product's epilogue stores each tile into every GPU's buffer
             over NVLink, then a barrier orders the ranks;
    nccl   = the product, an NCCL all-gather of the column blocks and the copy that places them."""
    import torch
    import torch.distributed as dist
    steps = max(1, min(args.steps, 10))
    flops = 2.0 * M * N * K
    rank = dist.get_rank()
    lo, hi = srt.shard_range(N, world, rank, 8)
    buf = srt.PeerBuffer((M, N), a.dtype)
    view = buf.tensor.narrow(1, lo, hi - lo)
    fused = srt.MatmulOp(view, a, False, b_full[:, lo:hi], False, peer_pointers=buf.peer_pointers(view))
    full = torch.empty((M, N), dtype=a.dtype, device=dev)

    def fused_step():
        fused()
        buf.ranks_done()

    def nccl_step():
        srt.sharded_matmul(a, b_full, axis="n", gather=True, out=full)

    # the same through an NVLink multicast mapping: each tile leaves the GPU once, the switch replicates it
    try:
        mbuf = srt.PeerBuffer((M, N), a.dtype, multicast=True)
    except Exception:                 # no symmetric memory on this machine: the per-peer form only
        mbuf = srt.PeerBuffer((M, N), a.dtype)
    mview = mbuf.tensor.narrow(1, lo, hi - lo)
    legs = [("fused", fused_step), ("nccl", nccl_step)]
    if mbuf.multicast_base:
        mc_op = srt.MatmulOp(mview, a, False, b_full[:, lo:hi], False, multicast_pointer=mbuf.multicast_pointer(mview))

        def multicast_step():
            mc_op()
            mbuf.ranks_done()
        legs.insert(1, ("fused_multicast", multicast_step))

    out = {"steps": steps, "bytes_sent_per_rank": int((world - 1) * M * (hi - lo) * a.element_size())}
    for name, fn in legs:
        for _ in range(3):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item()) / steps
        out[name + "_ms"] = ms
        out[name + "_tflops"] = flops / (ms * 1e-3) / 1e12
    status = srt.check_status()
    same = torch.equal(buf.tensor, full) and (not mbuf.multicast_base or torch.equal(mbuf.tensor, full))
    flag = torch.tensor([1 if (same and status == 0) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out["results_identical"] = bool(int(flag.item()))
    mbuf.close()
    buf.close()
    return out


# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import swiftrt_b200 as srt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    M, N, K, dtype, desc = WORKLOADS[args.workload]
    tdt = torch.bfloat16
    lo, hi = srt.shard_range(N, world, rank, 8)
    n_local = hi - lo
    g = torch.Generator(device=dev).manual_seed(0)
    a = (torch.rand((M, K), device=dev, generator=g) * 2 - 1).to(tdt)
    # every rank draws the same full B and keeps its column block as a strided view
    b_full = (torch.rand((K, N), device=dev, generator=g) * 2 - 1).to(tdt)
    b = b_full[:, lo:hi]
    c = torch.empty((M, n_local), dtype=tdt, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        srt.matmul_into(c, a, False, b, False)

    if args.tune:
        srt.set_tuning(*[int(x) for x in args.tune.split(",")])
    plan = srt.query_plan(a, b, c)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()          # nvidia-smi needs ~0.1 s to deliver its first sample: start it early
    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = srt.launch_count()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    events[0].record()
    for i in range(args.steps):
        step()
        events[i + 1].record()
    barrier()
    total_ms = events[0].elapsed_time(events[-1])
    launches = srt.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    status = srt.check_status()
    if status != 0:
        raise SystemExit(f"tensor-core kernel reported pipeline status {status}")
    kernel_ms = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    flops = 2.0 * M * N * K
    value = flops / (ms_per_step * 1e-3) / 1e12

    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(args, srt, a, b, M, N, K, n_local, dev, world, barrier)

    gather = None
    if world > 1 and not args.no_gather:
        try:
            gather = measure_gather(args, srt, a, b_full, M, N, K, dev, world, barrier)
        except Exception as e:        # the headline numbers above stand without this leg
            gather = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        pk, pk_kind = peaks()
        avg_kernel_ms = sum(kernel_ms) / len(kernel_ms)
        flops_launch = 2.0 * M * n_local * K
        achieved = flops_launch / (avg_kernel_ms * 1e-3) / 1e12
        peak = float(pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        # DRAM bytes per launch of this kernel on this workload from one ncu capture (dram__bytes_read.sum +
        # dram__bytes_write.sum, a one-pass metric pair; see profiles/): known for the unsharded 16384^3 case only
        traffic = 9.38e9 if (world == 1 and args.workload == "bf16_16384" and plan["kernel"] == 3 and not args.tune) else None
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": traffic, "peak_source": f"{pk_kind} cuBLAS bf16 burst", "frac_of_nominal_2250": achieved / 2250.0,
                    "kernel": {3: "gemm_tcgen05_pair_kernel", 2: "gemm_tcgen05_kernel", 1: "gemm_simt_kernel"}[plan["kernel"]],
                    "kernel_ms": avg_kernel_ms}
        # the timed region is back-to-back launches under the power cap: the sustained cuBLAS figure
        # (seconds-long loop) is the like-for-like companion of the burst one used for `frac`
        sustained = float(pk.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        roofline["peak_sustained"] = sustained
        roofline["frac_of_sustained"] = achieved / sustained
        line = {
            "metric": "GEMM TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": desc, "M": M, "N": N, "K": K, "sharding": f"N over {world} rank(s), no collective",
                       "l2": "inputs (512 MiB each) larger than the 126 MB L2", "plan": plan},
            "roofline": roofline,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "gather": gather,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            tf, cores, sample, _ = cpu_sample(M, N, K, cpu_inputs(N, K), target_s=args.cpu_seconds)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries print to stdout too (NCCL writes its version banner there), and the one JSON line
    must be the only thing on it: point fd 1 at stderr for the run and keep the real stdout aside."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    text = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    os.write(_RESULT_FD if _RESULT_FD is not None else 1, text)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="bf16_16384")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU time budget of the bounded CPU sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-gather", action="store_true", help="N > 1: skip the full-C-on-every-GPU comparison")
    ap.add_argument("--tune", default="", help="forceKernel,tileN,stages,maxCtas for srtMatmulSetTuning (0 = automatic)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    keep_stdout_for_the_result()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
