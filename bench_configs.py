"""Times the five named configurations of the matmul path on one GPU and prints one JSON record
per configuration (shape, kernel, ms, algorithmic TFLOP/s and GB/s, roofline fractions).

    python bench_configs.py [--iters 20] [--only c3]

Inputs are seeded synthetic draws with the shapes and value distributions of the configurations;
between timed launches a buffer larger than the L2 cache is read (not written: dirty lines would
make the timed kernel pay for their write-back), so every launch starts with a cold, clean L2.
Timing: CUDA events around each launch on the launching stream (the launch is a prepared
MatmulOp, enqueued while the flush still runs, so host latency is not in the interval), median
and best of `iters` after 3 warm-ups.
"""
from __future__ import annotations

import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import swiftrt_b200 as srt  # noqa: E402

NOMINAL = {"bf16_tflops": 2250.0, "hbm_gbs": 8000.0}
KERNEL_NAMES = {1: "gemm_simt_kernel", 2: "gemm_tcgen05_kernel", 3: "gemm_tcgen05_pair_kernel",
                4: "gemm_tcgen05_split_kernel"}


def measured_peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


def _uniform(shape, dtype, dev, g, lo, hi):
    return (torch.rand(shape, device=dev, generator=g) * (hi - lo) + lo).to(dtype)


def configs(dev):
    g = torch.Generator(device=dev).manual_seed(0)
    f32, f16, bf16 = torch.float32, torch.float16, torch.bfloat16

    def c1():
        return dict(name="c1", desc="Float32 256^3 NN", a=_uniform((256, 256), f32, dev, g, -1, 1),
                    b=_uniform((256, 256), f32, dev, g, -1, 1), bound="hbm")

    def c2():
        return dict(name="c2", desc="Dense bf16 [1024x4096].[4096x4096] + bias, ReLU",
                    a=_uniform((1024, 4096), bf16, dev, g, -0.05, 0.05), b=_uniform((4096, 4096), bf16, dev, g, -0.05, 0.05),
                    bias=_uniform((4096,), bf16, dev, g, -0.05, 0.05), act=srt.ActivationType.relu, bound="tensor")

    def c3():
        return dict(name="c3", desc="batched fp16 64 x [512x64].[512x64]^T",
                    a=torch.randn((64, 512, 64), device=dev, generator=g).to(f16),
                    b=torch.randn((64, 512, 64), device=dev, generator=g).to(f16), tb=True, bound="hbm")

    def c4():
        return dict(name="c4", desc="Float32 [65536x1024].[1024x256] NN", a=_uniform((65536, 1024), f32, dev, g, -1, 1),
                    b=_uniform((1024, 256), f32, dev, g, -1, 1), bound="hbm")

    def c5():
        return dict(name="c5", desc="bf16 16384^3 NN", a=_uniform((16384, 16384), bf16, dev, g, -1, 1),
                    b=_uniform((16384, 16384), bf16, dev, g, -1, 1), bound="tensor")

    return [c1, c2, c3, c4, c5]


def run(cfg: dict, iters: int, flush: torch.Tensor, peaks: dict, autotune: bool = False) -> dict:
    sink = torch.zeros((), dtype=torch.float32, device=flush.device)
    a, b = cfg["a"], cfg["b"]
    tb = cfg.get("tb", False)
    bias, act = cfg.get("bias"), cfg.get("act")
    out = srt.matmul(a, b, False, tb, bias=bias, activation=act)
    if autotune:
        srt.tune(a, b, out, False, tb, bias, act)           # the fastest candidate (warm L2) goes into the plan table
    plan = srt.query_plan(a, b, out, False, tb)
    op = srt.MatmulOp(out, a, False, b, tb, bias, act)
    for _ in range(3):
        op()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        sink.copy_(flush.sum())                         # evicts L2 with clean lines: 256 MiB read
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        op()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    if srt.check_status() != 0:
        raise RuntimeError("tensor-core kernel reported a pipeline timeout")
    times.sort()
    med, best = times[len(times) // 2], times[0]
    batch = a.shape[0] if a.dim() == 3 else 1
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-2] if tb else b.shape[-1]
    flops = 2.0 * batch * M * N * K
    nbytes = (a.numel() + b.numel() + out.numel()) * a.element_size() + (bias.numel() * bias.element_size() if bias is not None else 0)
    tf, gbs = flops / med / 1e9, nbytes / med / 1e6
    rec = {"config": cfg["name"], "what": cfg["desc"], "kernel": KERNEL_NAMES[plan["kernel"]],
           "tile": [plan["tileM"], plan["tileN"], plan["tileK"]], "stages": plan["stages"], "ctas": plan["ctas"],
           "ms_median": med, "ms_best": best, "algorithmic_flops": flops, "algorithmic_bytes": nbytes,
           "tflops": tf, "gbs": gbs, "bound": cfg["bound"]}
    if cfg["bound"] == "tensor":
        rec["frac_of_nominal"] = tf / NOMINAL["bf16_tflops"]
        if "bf16_tflops" in peaks:
            rec["frac_of_measured"] = tf / peaks["bf16_tflops"]
    else:
        rec["frac_of_nominal"] = gbs / NOMINAL["hbm_gbs"]
        if "hbm_gbs" in peaks:
            rec["frac_of_measured"] = gbs / peaks["hbm_gbs"]
    return rec


def _time_cold(fn, iters: int, flush: torch.Tensor) -> tuple[float, float]:
    """Median and best device time (ms) of fn() after an L2 flush, over `iters` runs."""
    sink = torch.zeros((), dtype=torch.float32, device=flush.device)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        sink.copy_(flush.sum())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2], times[0]


def run_backward(dev, iters: int, flush: torch.Tensor, peaks: dict, rows: int = 16384, cols: int = 8192) -> dict:
    """f1: srtBiasActivationBackward, bf16 [rows x cols], ReLU: reads dy and y, writes dz (+ column sums)."""
    g = torch.Generator(device=dev).manual_seed(0)
    dy = torch.randn((rows, cols), device=dev, generator=g).to(torch.bfloat16)
    y = torch.relu(torch.randn((rows, cols), device=dev, generator=g)).to(torch.bfloat16)
    med, best = _time_cold(lambda: srt.bias_activation_backward(dy, y, srt.ActivationType.relu), iters, flush)
    nbytes = 3 * dy.numel() * 2 + cols * 2
    rec = {"config": "f1", "what": f"bias/activation backward bf16 [{rows}x{cols}] ReLU (dz and dbias)",
           "kernel": "dense_backward_kernel + dense_backward_finish_kernel", "ms_median": med, "ms_best": best,
           "algorithmic_bytes": nbytes, "gbs": nbytes / med / 1e6, "bound": "hbm", "frac_of_nominal": nbytes / med / 1e6 / NOMINAL["hbm_gbs"]}
    if "hbm_gbs" in peaks:
        rec["frac_of_measured"] = rec["gbs"] / peaks["hbm_gbs"]
    return rec


def run_lstm(dev, iters: int, flush: torch.Tensor, peaks: dict, batch: int = 4096, nx: int = 1024, nh: int = 1024) -> dict:
    """f4: one LSTM cell step, bf16: concatenation, fused product [batch x (nx+nh)].[(nx+nh) x 4nh] + bias, gate pass."""
    g = torch.Generator(device=dev).manual_seed(0)
    bf16 = torch.bfloat16
    x = _uniform((batch, nx), bf16, dev, g, -1, 1)
    state = srt.LSTMState(_uniform((batch, nh), bf16, dev, g, -1, 1), _uniform((batch, nh), bf16, dev, g, -1, 1))
    cell = srt.LSTMCell(_uniform((nx + nh, 4 * nh), bf16, dev, g, -0.03, 0.03), _uniform((4 * nh,), bf16, dev, g, -0.5, 0.5))
    med, best = _time_cold(lambda: cell(x, state), iters, flush)
    fused_cell = srt.LSTMCell(cell.fused_weight, cell.fused_bias, fuse_gates=True)
    fused_med, _ = _time_cold(lambda: fused_cell(x, state), iters, flush)
    flops = 2.0 * batch * (nx + nh) * 4 * nh
    # each tensor once: x, h, c, W, b in; c', h' out (the concatenated input and the fused product are intermediates)
    nbytes = 2 * (batch * nx + 2 * batch * nh + (nx + nh) * 4 * nh + 4 * nh + 2 * batch * nh)
    rec = {"config": "f4", "what": f"LSTM cell step bf16 batch {batch}, input {nx}, hidden {nh}",
           "kernel": "concat_kernel + gemm + lstm_gates_kernel", "ms_median": med, "ms_best": best,
           "gates_in_epilogue_ms_median": fused_med,
           "algorithmic_flops": flops, "algorithmic_bytes": nbytes, "tflops": flops / med / 1e9, "gbs": nbytes / med / 1e6,
           "bound": "tensor", "frac_of_nominal": flops / med / 1e9 / NOMINAL["bf16_tflops"]}
    if "bf16_tflops" in peaks:
        rec["frac_of_measured"] = rec["tflops"] / peaks["bf16_tflops"]
    return rec


def run_small_batch(dev, iters: int, flush: torch.Tensor, peaks: dict) -> list:
    """s1: a few rows through a 4096 x 4096 Dense layer (bias + ReLU), bf16, cold L2; the same with
    torch.addmm + ReLU (cuBLAS) beside it."""
    g = torch.Generator(device=dev).manual_seed(0)
    bf16 = torch.bfloat16
    w = _uniform((4096, 4096), bf16, dev, g, -0.5, 0.5)
    b = _uniform((4096,), bf16, dev, g, -0.5, 0.5)
    out = []
    for rows in (1, 8, 32, 64, 128, 256):
        x = _uniform((rows, 4096), bf16, dev, g, -0.5, 0.5)
        y = torch.empty((rows, 4096), dtype=bf16, device=dev)
        op = srt.MatmulOp(y, x, False, w, False, b, srt.ActivationType.relu)
        plan = srt.query_plan(x, w, y)
        med, best = _time_cold(op, iters, flush)
        t_med, _ = _time_cold(lambda: torch.relu_(torch.addmm(b, x, w)), iters, flush)
        nbytes = (x.numel() + w.numel() + y.numel() + b.numel()) * 2
        rec = {"config": "s1", "what": f"Dense bf16 [{rows}x4096].[4096x4096] + bias, ReLU", "kernel": KERNEL_NAMES[plan["kernel"]],
               "tile": [plan["tileM"], plan["tileN"], plan["tileK"]], "transposed_plan": bool(plan["swapped"]), "splitK": plan["splitK"],
               "ms_median": med, "ms_best": best, "algorithmic_bytes": nbytes, "gbs": nbytes / med / 1e6, "bound": "hbm",
               "torch_addmm_relu_ms": t_med}
        if "hbm_gbs" in peaks:
            rec["frac_of_measured"] = rec["gbs"] / peaks["hbm_gbs"]
        out.append(rec)
    return out


def run_transform(dev, iters: int, flush: torch.Tensor, peaks: dict) -> list:
    """t1: srtMatrixTransform re-layouts (one read and one write per element): HBM-bound byte shuffles."""
    out = []
    D, O = srt.DataType, srt.Order
    cases = [("int8 16384x16384 row -> colTiledTC32x32", D.real8I, 16384, 16384, O.row, O.colTiledTC32x32),
             ("int8 16384x16384 colTiledTC32x32 -> row", D.real8I, 16384, 16384, O.colTiledTC32x32, O.row),
             ("bf16 16384x8192 row -> colTiled32", D.real16BF, 16384, 8192, O.row, O.colTiled32),
             ("int8 16384x16384 col -> colTiledTC32x32 (transposition)", D.real8I, 16384, 16384, O.col, O.colTiledTC32x32),
             ("fp32 8192x8192 row -> col (transpose)", D.real32F, 8192, 8192, O.row, O.col),
             ("fp32 8192x8192 row -> row (copy)", D.real32F, 8192, 8192, O.row, O.row)]
    for what, dtype, rows, cols, src, dst in cases + [("fp32 row -> int8 colTiledTC32x32 16384x8192, alpha = 0.5 (quantise)", D.real32F, 16384, 8192, O.row, O.colTiledTC32x32)]:
        quantise = "quantise" in what
        la, lc = srt.MatrixLayout(dtype, src, rows, cols), srt.MatrixLayout(D.real8I if quantise else dtype, dst, rows, cols)
        a = la.empty(dev)
        if dtype == D.real8I:
            a.random_(-128, 128)
        else:
            a.normal_()
        c = lc.empty(dev)
        med, best = _time_cold(lambda: srt.matrix_transform(a, la, lc, alpha=0.5 if quantise else 1.0, out=c), iters, flush)
        nbytes = rows * cols * (a.element_size() + c.element_size())
        rec = {"config": "t1", "what": what, "kernel": "matrix_transform_kernel", "ms_median": med, "ms_best": best,
               "algorithmic_bytes": nbytes, "gbs": nbytes / med / 1e6, "bound": "hbm", "frac_of_nominal": nbytes / med / 1e6 / NOMINAL["hbm_gbs"]}
        if "hbm_gbs" in peaks:
            rec["frac_of_measured"] = rec["gbs"] / peaks["hbm_gbs"]
        out.append(rec)
        del a, c
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="")
    ap.add_argument("--tune", default="", help="forceKernel,tileN,stages,maxCtas")
    ap.add_argument("--autotune", action="store_true", help="run srtMatmulTune on each configuration first")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if args.tune:
        srt.set_tuning(*[int(x) for x in args.tune.split(",")])
    flush = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    peaks = measured_peaks()
    only = args.only.split(",") if args.only else []
    # the callers either side of the product and the small-batch Dense shapes are measured on request only (--only f1,f4,s1,t1)
    if "f1" in only:
        print(json.dumps(run_backward(dev, args.iters, flush, peaks)), flush=True)
    if "f4" in only:
        print(json.dumps(run_lstm(dev, args.iters, flush, peaks)), flush=True)
    if "s1" in only:
        for rec in run_small_batch(dev, args.iters, flush, peaks):
            print(json.dumps(rec), flush=True)
    if "t1" in only:
        for rec in run_transform(dev, args.iters, flush, peaks):
            print(json.dumps(rec), flush=True)
    for make in configs(dev):
        if only and make.__name__ not in only:
            continue
        cfg = make()
        print(json.dumps(run(cfg, args.iters, flush, peaks, args.autotune)), flush=True)
        del cfg
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
