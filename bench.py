#!/usr/bin/env python
"""Benchmark of the Winograd-ReLU F(2x2,3x3) convolution path on B200, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--math tf32|fp32]
                    [--workload cfg2|cfg1|cfg3|cfg4|cfg5] [--layout NCHW|NHWC] [--only-headline]

Prints ONE JSON line (rank 0).  The headline (`value`, `ms_per_step`, `roofline`, `e2e`) is the layer forward
of the conv2_x-shaped workload (N=64, C=K=64, 56x56, dense): `value` with inputs resident in HBM, timed over
`--steps` launches back to back between two CUDA events; `e2e` the same through the host-buffer call (H2D of
X and D2H of Y inside the timed region); `roofline` for the dominant kernel, whose duration comes from a
separate short pass after the timed region.  `configs` holds one sub-record per other workload, each measured
in this run with its own step count: cfg1 (N=4 layer), cfg3 (pruned conv4_x-shaped layer forward, with the
zero-block skip rate of its mask), cfg5 (conv5_x-shaped layer backward on the tensor cores) and cfg4
(ResNet-18-var forward, batch 256 in total: sharded over the ranks under --gpus N, replayed as a CUDA graph,
with the NCCL all-gather of the logits timed beside it).  `cpu_baseline` is the C restatement of the layer
math on the host cores; `reference_gpu` is the reference's own CUDA kernels (compiled unmodified for sm_100a
by oracle/Makefile) on the headline workload.  `--impl reference` times the C restatement (the reference has
no CPU implementation of its own: its CPU kernels exit).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "sparse-winograd-cnn_b200"))

WORKLOADS = {  # per-GPU shapes: B, C, K, H, W, weight density, post-ReLU input
    "cfg1": dict(B=4, C=64, K=64, H=56, W=56, density=1.0, halfnormal=False),
    "cfg2": dict(B=64, C=64, K=64, H=56, W=56, density=1.0, halfnormal=False),
    "cfg3": dict(B=128, C=256, K=256, H=14, W=14, density=0.3, halfnormal=True),
}
CFG5 = dict(B=256, C=512, K=512, H=7, W=7, density=0.2)
METRIC = "winograd_relu_conv_layer_fwd_throughput"
UNIT = "img/s"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the one-pass ncu captures summarised under
# profiles/ (taken at the workload's full size); a constant from those captures, not a per-run measurement
NCU_TRAFFIC = {
    ("cfg2", 64, "NCHW", "imtrans"): (197.8e6, "ncu capture, profiles/imtrans_fwd_nchw_band_kernel_cfg2.md"),
    ("cfg2", 64, "NCHW", "conv"): (224.7e6, "ncu capture, profiles/conv_fwd_tc_kernel_cfg2.md"),
    ("cfg2", 64, "NCHW", "fused"): (60.0e6, "ncu capture, profiles/layer_fwd_fused_kernel_cfg2.md (X read once; most of Y is still "
                                            "dirty in L2 when the launch ends, so it is below the algorithmic X + W + Y)"),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def make_inputs(wl, seed=1):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((wl["B"], wl["C"], wl["H"], wl["W"]), dtype=np.float32)
    if wl["halfnormal"]:
        X = np.maximum(X, 0)
    rw = np.random.default_rng(2)
    Wt = (0.05 * rw.standard_normal((16, wl["C"], wl["K"]))).astype(np.float32)
    if wl["density"] < 1.0:
        Wt *= (np.random.default_rng(3).random(Wt.shape) < wl["density"]).astype(np.float32)
    return X, Wt


class ClockSampler:
    """`nvidia-smi -lms 20` running beside the benchmark; rows are stamped on arrival so that the ones that
    fall inside the timed region can be picked out afterwards."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.rows = []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 6:
                self.rows.append((time.time(), f))

    def finish(self, t0, t1):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        time.sleep(0.12)
        self.proc.terminate()
        inside = [f for (t, f) in self.rows if t0 <= t <= t1 + 0.06]
        window = "timed region"
        if len(inside) < 2:   # region shorter than the sampling period: take the whole run (warm-up included)
            inside, window = [f for (_, f) in self.rows], "whole run"
        sm = [float(f[0]) for f in inside if f[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for f in inside for n, v in zip(names, f[2:6]) if v.lower().startswith("active")})
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=float(inside[0][1]) if inside else None,
                    reasons=reasons, samples=len(inside), window=window)


# ---------------------------------------------------------------------------------------------------------
# CPU legs (the only places where this file runs anything under oracle/)
# ---------------------------------------------------------------------------------------------------------
def _fwd_port(wl, b):
    """A callable that runs the C restatement of the layer forward once on a batch slice of b images."""
    from oracle import wg_oracle as o
    X, Wt = make_inputs(dict(wl, B=b))
    Xn = np.ascontiguousarray(np.transpose(X, (0, 2, 3, 1)))
    P = b * ((wl["H"] + 1) // 2) * ((wl["W"] + 1) // 2)
    bufs = (np.empty((b, wl["H"], wl["W"], wl["K"]), np.float32), np.empty(16 * P * wl["C"], np.float32),
            np.empty(16 * P * wl["K"], np.float32))
    return lambda: o.layer_fwd(Xn, Wt, relu=True, dtype=np.float32, bufs=bufs)


def _bwd_port(b):
    """The C restatement of the conv5_x-shaped backward (wgo_conv_bwd + wgo_imtrans_bwd with the ReLU mask) on b images."""
    from oracle import wg_oracle as o
    C, K, H, W = CFG5["C"], CFG5["K"], CFG5["H"], CFG5["W"]
    rng = np.random.default_rng(1)
    X = rng.standard_normal((b, H, W, C), dtype=np.float32)
    mask = (np.random.default_rng(3).random((16, C, K)) < CFG5["density"]).astype(np.float32)
    Wt = (0.05 * np.random.default_rng(2).standard_normal((16, C, K))).astype(np.float32) * mask
    dY = rng.standard_normal((b, H, W, K), dtype=np.float32)
    V = o.imtrans_fwd(X, relu=True, dtype=np.float32)

    def run():
        dV, dW = o.conv_bwd(V, Wt, dY, mask=mask, dtype=np.float32)
        return o.imtrans_bwd(dV, H, W, Vmask=V, dtype=np.float32), dW
    return run


def _time_cpu(fn, seconds):
    fn()   # warm
    n, t0 = 0, time.perf_counter()
    while True:
        fn()
        n += 1
        dt = time.perf_counter() - t0
        if dt > seconds:
            return n, dt


def cpu_baseline(wl, seconds=10.0):
    """Images per second of the C restatement (float32, OpenMP over all host cores) on a batch slice."""
    from oracle import wg_oracle as o
    cores = o.set_threads()
    b = max(1, min(wl["B"], 4))
    n, dt = _time_cpu(_fwd_port(wl, b), seconds)
    return dict(value=b * n / dt, unit=UNIT, cores=cores, kind="port",
                sample="batch slice of %d images of the %dx%dx%dx%d layer forward, %d passes in %.1f s, float32 C restatement with OpenMP"
                       % (b, wl["C"], wl["K"], wl["H"], wl["W"], n, dt))


def cpu_baseline_bwd(seconds=6.0):
    from oracle import wg_oracle as o
    cores = o.set_threads()
    b = 4
    n, dt = _time_cpu(_bwd_port(b), seconds)
    return dict(value=b * n / dt, unit=UNIT, cores=cores, kind="port",
                sample="batch slice of %d images of the 512x512x7x7 layer backward (dV, masked dW, dX with the ReLU mask), %d passes in "
                       "%.1f s, float32 C restatement with OpenMP" % (b, n, dt))


def run_reference(args, rank):
    """--impl reference: the reference layer math on the host cores.  The reference ships GPU-only ops (its CPU
    kernels print and exit), so this arm is the C restatement under oracle/ on a bounded batch slice."""
    if rank != 0:
        return
    from oracle import wg_oracle as o
    cores = o.set_threads()
    if args.workload == "cfg4":
        # the network's 16 Winograd-ReLU layers, one image each, summed (the dense parts of the network -- stem, pools,
        # 1x1 shortcuts, FC -- are stock ops in the reference too and are left out)
        shapes = [(64, 64, 56, 4), (64, 128, 28, 1), (128, 128, 28, 3), (128, 256, 14, 1), (256, 256, 14, 3),
                  (256, 512, 7, 1), (512, 512, 7, 3)]
        fns = [(_fwd_port(dict(C=c, K=k, H=s, W=s, density=1.0, halfnormal=False), 1), rep) for c, k, s, rep in shapes]
        b, metric = 1, "resnet18_var_forward_throughput"
        step = lambda: [f() for f, rep in fns for _ in range(rep)]
        sample = "each step = the 16 Winograd-ReLU layers of the network on one image (host cores, OpenMP, float32); dense layers left out"
        cfg = {"workload": "cfg4", "sample_batch": 1}
    elif args.workload == "cfg5":
        b, metric = 4, "winograd_relu_conv_layer_bwd_throughput"
        step = _bwd_port(b)
        sample = "each step = batch slice of %d images of the backward workload (host cores, OpenMP, float32)" % b
        cfg = {"workload": "cfg5", "layer": CFG5, "layout": "NHWC", "sample_batch": b}
    else:
        wl = dict(WORKLOADS[args.workload])
        b, metric = max(1, min(wl["B"], 4)), METRIC
        step = _fwd_port(wl, b)
        sample = "each step = batch slice of %d images of the workload (host cores, OpenMP, float32)" % b
        cfg = {"workload": args.workload, "layer": wl, "layout": "NHWC", "sample_batch": b}
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = b * args.steps / dt
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": "strong" if args.workload == "cfg4" else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg, "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference ships GPU-only ops (its CPU kernels exit); this arm is the C restatement of its layer math",
    }))


# ---------------------------------------------------------------------------------------------------------
# GPU helpers
# ---------------------------------------------------------------------------------------------------------
class Ctx:
    """Rank, device and the collective plumbing shared by the GPU workloads."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
            dist.barrier()      # builds the communicator now, so that the barrier in front of a timed region is only a barrier

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, ms):
        if self.world == 1:
            return float(ms)
        t = self.torch.tensor([ms], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed(ctx, fn, steps, warmup=3):
    """ms per call of fn(i): `warmup` untimed calls, then `steps` calls back to back between two CUDA events on the
    launching stream, barrier + synchronize on both sides, max over ranks."""
    torch = ctx.torch
    for i in range(warmup):
        fn(i)
    ctx.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        fn(i)
    b.record()
    ctx.barrier()
    return ctx.max_over_ranks(a.elapsed_time(b)) / steps


def each_launch_ms(torch, fn, n):
    """Mean duration of fn(i) with every call bracketed by its own pair of events (no overlap with its neighbours)."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for i in range(n):
        ev[i][0].record()
        fn(i)
        ev[i][1].record()
    torch.cuda.synchronize()
    return float(np.mean([a.elapsed_time(b) for a, b in ev]))


def check_status(wg2x2):
    status, where = wg2x2.last_device_status()
    if status != 0:
        raise RuntimeError("device status %d at 0x%x" % (status, where))


class LayerFwd:
    """One Winograd-ReLU layer forward on rotating input buffers (inputs + outputs of consecutive steps exceed L2)."""

    def __init__(self, ctx, wl, layout, math, path, nbuf=4):
        import wg2x2
        torch = ctx.torch
        self.wg, self.ctx, self.wl, self.layout, self.math = wg2x2, ctx, wl, layout, math
        B, C, K, H, W = wl["B"], wl["C"], wl["K"], wl["H"], wl["W"]
        nH, nW = (H + 1) // 2, (W + 1) // 2
        self.P = B * nH * nW
        Xh, Wth = make_inputs(wl, seed=1 + ctx.rank)
        if layout == "NHWC":
            Xh = np.ascontiguousarray(np.transpose(Xh, (0, 2, 3, 1)))
        self.Xh, self.Wth = Xh, Wth
        # enough rotating inputs that what a step touches has left L2 (126 MB) when its buffer comes round again
        while nbuf * Xh.nbytes < 200e6 and nbuf < 16:
            nbuf += 1
        self.nbuf = nbuf
        self.Xs = [torch.from_numpy(Xh).to(ctx.dev) + 0.0 * i for i in range(nbuf)]
        self.Wt = torch.from_numpy(Wth).to(ctx.dev)
        self.V = torch.empty((16, B, nH, nW, C), device=ctx.dev)
        self.Y = torch.empty((B, K, H, W) if layout == "NCHW" else (B, H, W, K), device=ctx.dev)
        lib = wg2x2._lib.lib
        ws_n = lib.wg2x2_conv_fwd_workspace_bytes(B, nH, nW, C, K, wg2x2.ops._MATHS[math])
        self.ws = torch.empty(max(ws_n, 1), dtype=torch.uint8, device=ctx.dev)
        # the weights do not change between forward passes: the tensor-core path repacks them once
        self.prepared = wg2x2.prepare_weights(self.Wt) if math == "tf32" else None
        cws_n = lib.wg2x2_conv_fwd_prepared_workspace_bytes(B, nH, nW, C, K) if self.prepared is not None else 0
        self.cws = torch.empty(cws_n, dtype=torch.uint8, device=ctx.dev) if cws_n else None   # products of the wide path (C, K >= 256)
        fused_ok = self.prepared is not None and layout == "NCHW" and wg2x2.fused_supported(B, H, W, C, K, "NCHW")
        fused_pays = K <= 128 or (K <= 256 and C <= 64)          # the library's own rule (wg2x2_layer_fwd_prepared)
        self.use_fused = fused_ok and (path == "fused" or (path == "auto" and fused_pays))
        self.bytesX, self.bytesV, self.bytesY, self.bytesW = 4 * B * C * H * W, 64 * self.P * C, 4 * B * K * H * W, 64 * C * K
        self.flops = 2.0 * 16 * self.P * C * K
        self._fused_calls = None

    def imtrans(self, i):
        self.wg.imtrans_fwd(self.Xs[i % self.nbuf], relu=True, layout=self.layout, out=self.V)

    def conv(self, i):
        wl = self.wl
        if self.prepared is not None:
            self.wg.conv_fwd_prepared(self.V, self.prepared, wl["K"], wl["H"], wl["W"], layout=self.layout, out=self.Y, workspace=self.cws)
        else:
            self.wg.conv_fwd(self.V, self.Wt, wl["H"], wl["W"], layout=self.layout, math=self.math, out=self.Y, workspace=self.ws)

    def fused(self, i):
        # straight through the C ABI with the arguments built once: the timed loop is one foreign call per step, as in the
        # reference's op Compute (the Python wrapper's argument checks would cost a third of a 47 us step on the host)
        if self._fused_calls is None:
            lib = self.wg._lib.lib
            wl = self.wl
            stream = ctypes.c_void_p(self.ctx.torch.cuda.current_stream().cuda_stream)
            P = ctypes.c_void_p
            self._fused_calls = [
                (lib.wg2x2_layer_fwd_fused, (P(x.data_ptr()), P(self.prepared.data_ptr()), P(self.Y.data_ptr()), wl["B"], wl["H"], wl["W"],
                                             wl["C"], wl["K"], 1, None, None, None, stream)) for x in self.Xs]
        fn, a = self._fused_calls[i % self.nbuf]
        rc = fn(*a)
        if rc != 0:
            raise RuntimeError("wg2x2_layer_fwd_fused returned %d" % rc)

    def step(self, i):
        if self.use_fused:
            self.fused(i)
        else:
            self.imtrans(i)
            self.conv(i)

    def layer_bytes(self):
        return self.bytesX + self.bytesW + self.bytesY if self.use_fused else 2 * self.bytesV + self.bytesX + self.bytesW + self.bytesY

    def roofline(self, pk, n_each=24):
        """Per-kernel durations from a separate pass (each launch bracketed by its own events) and the roofline of
        the dominant kernel: algorithmic bytes or flops of one launch / its duration, against the measured peak."""
        torch = self.ctx.torch
        tf32_peak = pk["bf16_tflops"] / 2.0
        k1_bytes, k2_bytes = self.bytesX + self.bytesV, self.bytesV + self.bytesW + self.bytesY
        if self.use_fused:
            ms = each_launch_ms(torch, self.fused, n_each)
            fb = self.bytesX + self.bytesW + self.bytesY
            roof = dict(kernel="layer_fwd_fused_kernel (transform + ReLU + products + output transform, one launch = the whole layer)",
                        bound="hbm", achieved=fb / (ms * 1e-3) / 1e9, peak=pk["hbm_gbs"], unit="GB/s", peak_source=pk["source"],
                        algorithmic_bytes=fb, tensor_tflops_algorithmic=self.flops / (ms * 1e-3) / 1e12,
                        tensor_tflops_issued=2.25 * self.flops / (ms * 1e-3) / 1e12, kernels_ms={"layer_fwd_fused": ms},
                        note="only X, W and Y cross HBM; the kernel is paced by the SM, not by HBM (36 signed MMAs per 8 channels instead "
                             "of 16, transform warps in step with them).  kernels_ms is a launch bracketed by events on its own; back to "
                             "back the launches overlap their neighbours' tails (programmatic dependent launch), so ms_per_step can be below it")
            which = "fused"
        else:
            ms1 = each_launch_ms(torch, self.imtrans, n_each)
            ms2 = each_launch_ms(torch, self.conv, n_each)
            t_hbm, t_tensor = k2_bytes / (pk["hbm_gbs"] * 1e9), self.flops / (tf32_peak * 1e12)
            if ms2 >= ms1:
                which = "conv"
                if self.math == "tf32" and t_tensor > t_hbm:
                    roof = dict(kernel="conv_fwd (the 16 products + output transform)", bound="tensor", achieved=self.flops / (ms2 * 1e-3) / 1e12,
                                peak=tf32_peak, unit="TFLOP/s", peak_source=pk["source"] + " bf16 / 2", algorithmic_flops=self.flops)
                else:
                    roof = dict(kernel="conv_fwd (the 16 products + output transform)", bound="hbm", achieved=k2_bytes / (ms2 * 1e-3) / 1e9,
                                peak=pk["hbm_gbs"], unit="GB/s", peak_source=pk["source"], algorithmic_bytes=k2_bytes)
            else:
                which = "imtrans"
                roof = dict(kernel="imtrans_fwd (input transform + ReLU)", bound="hbm", achieved=k1_bytes / (ms1 * 1e-3) / 1e9,
                            peak=pk["hbm_gbs"], unit="GB/s", peak_source=pk["source"], algorithmic_bytes=k1_bytes)
            roof["kernels_ms"] = {"imtrans_fwd": ms1, "conv_fwd": ms2}
            roof["imtrans_fwd_gbs"] = k1_bytes / (ms1 * 1e-3) / 1e9
            roof["conv_fwd_gbs"] = k2_bytes / (ms2 * 1e-3) / 1e9
            roof["conv_fwd_tflops"] = self.flops / (ms2 * 1e-3) / 1e12
        roof["frac"] = roof["achieved"] / roof["peak"]
        return roof, which


def library_tf32(ctx, shapes, n=12):
    """Calibration, not a product path: cuBLAS TF32 batched GEMMs (torch.bmm, allow_tf32) on the given (batch, M, K, N)
    products with resident operands and nothing else (no transforms, masks or epilogues) -- what the vendor library reaches
    on the same tensor-core shapes, beside the measured bf16 / 2 roof."""
    torch = ctx.torch
    keep = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        ops = [(torch.randn((b, m, k), device=ctx.dev), torch.randn((b, k, nn), device=ctx.dev)) for (b, m, k, nn) in shapes]
        outs = [torch.empty((b, m, nn), device=ctx.dev) for (b, m, k, nn) in shapes]

        def run(i):
            for (a, w), o in zip(ops, outs):
                torch.bmm(a, w, out=o)

        for i in range(3):
            run(i)
        ms = each_launch_ms(torch, run, n)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = keep
    flops = sum(2.0 * b * m * k * nn for (b, m, k, nn) in shapes)
    return {"what": "cuBLAS TF32 (torch.bmm) on the same products, operands resident, nothing else", "shapes_b_m_k_n": [list(x) for x in shapes],
            "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12}


def sub_layer_fwd(ctx, name, args, steps):
    """configs.<name>: one layer forward workload, device-resident."""
    wl = dict(WORKLOADS[name])
    L = LayerFwd(ctx, wl, "NCHW", "tf32", "auto")
    ms = timed(ctx, L.step, steps)
    check_status(L.wg)
    pk = peaks()
    roof, _ = L.roofline(pk, n_each=12)
    roof["traffic"] = None
    rec = {"ms_per_step": ms, "steps": steps, "img_s": ctx.world * wl["B"] / (ms * 1e-3), "layer": wl, "layout": "NCHW", "dtype": "tf32",
           "path": "one fused kernel" if L.use_fused else ("input transform, then products as GEMMs with 256 output channels per unit "
                                                          "into scratch + output transform pass" if L.cws is not None else "two kernels, V through HBM"),
           "layer_tflops": L.flops / (ms * 1e-3) / 1e12, "layer_gbs": L.layer_bytes() / (ms * 1e-3) / 1e9,
           "strict_layer_bound_ms": 1e3 * max((L.bytesX + L.bytesW + L.bytesY) / (pk["hbm_gbs"] * 1e9), L.flops / (pk["bf16_tflops"] / 2 * 1e12)),
           "roofline": roof}
    if wl["density"] < 1.0:
        from wg_weights import gen_prune_mask, zero_block_fraction
        rec["skip_rate"] = zero_block_fraction(L.Wth)           # share of 64 x 32 weight blocks that are all zero and skipped
        w2 = (0.05 * np.random.default_rng(2).standard_normal((16, wl["C"], wl["K"]))).astype(np.float32)
        rec["skip_rate_magnitude_mask"] = zero_block_fraction(gen_prune_mask(w2, wl["density"]))   # the reference's top-|w| mask, same density
        rec["skip_note"] = "unstructured masks leave no 64 x 32 block empty: tensor-pipe figures are from dense flops"
    if not L.use_fused and wl["C"] >= 256:       # tensor-bound shape: the vendor library's rate on the same 16 products, for scale
        P = wl["B"] * ((wl["H"] + 1) // 2) * ((wl["W"] + 1) // 2)
        rec["library_tf32"] = library_tf32(ctx, [(16, P, wl["C"], wl["K"])])
    del L
    ctx.torch.cuda.empty_cache()
    return rec


def sub_backward(ctx, args, steps, math="tf32", batch=0):
    """configs.cfg5: backward of the pruned conv5_x-shaped layer: dV and masked dW (gradient products), then dX through the
    input-transform gradient with the ReLU mask.  Per-GPU batch fixed."""
    import wg2x2
    torch = ctx.torch
    B, C, K, H, W = (batch or CFG5["B"]), CFG5["C"], CFG5["K"], CFG5["H"], CFG5["W"]
    nH = nW = 4
    P = B * nH * nW
    g = torch.Generator().manual_seed(1 + ctx.rank)
    X = torch.randn((B, C, H, W), generator=g).to(ctx.dev)
    mask = (torch.rand((16, C, K), generator=torch.Generator().manual_seed(3)) < CFG5["density"]).float().to(ctx.dev)
    Wt = (0.05 * torch.randn((16, C, K), generator=torch.Generator().manual_seed(2))).to(ctx.dev) * mask
    dYs = [torch.randn((B, K, H, W), generator=g).to(ctx.dev) for _ in range(2)]
    V = wg2x2.imtrans_fwd(X, relu=True, layout="NCHW")
    hold = {}

    def products(i):   # relu=True: the ReLU mask (V > 0) is applied in the dV product's epilogue, which runs beside the tensor pipe
        hold["dV"], hold["dW"] = wg2x2.conv_bwd(V, Wt, dYs[i % 2], mask=mask, layout="NCHW", relu=True, math=math)

    def gather(i):
        hold["dX"] = wg2x2.imtrans_bwd(hold["dV"], H, W, layout="NCHW")

    def step(i):
        products(i)
        gather(i)

    ms = timed(ctx, step, steps)
    check_status(wg2x2)
    ms_p = each_launch_ms(torch, products, 6)
    ms_g = each_launch_ms(torch, gather, 6)
    pk = peaks()
    flops = 2.0 * 2 * 16 * P * C * K
    bytes_alg = 4.0 * B * K * H * W + 64.0 * P * C + 2 * 64.0 * C * K + 4.0 * B * C * H * W + 64.0 * C * K
    tf32_peak = pk["bf16_tflops"] / 2
    from wg_weights import zero_block_fraction
    rec = {"ms_per_step": ms, "steps": steps, "img_s": ctx.world * B / (ms * 1e-3), "layer": dict(CFG5, B=B), "layout": "NCHW",
           "dtype": "tf32" if math == "tf32" else "f32", "layer_tflops": flops / (ms * 1e-3) / 1e12,
           "strict_layer_bound_ms": 1e3 * max(bytes_alg / (pk["hbm_gbs"] * 1e9), flops / (tf32_peak * 1e12)),
           "skip_rate": zero_block_fraction(mask.cpu().numpy()),
           "roofline": {"kernel": "conv_bwd (A dY A^T, dV = dM.W^T with the ReLU mask in its epilogue, dW = V^T.dM on the tensor cores) + imtrans_bwd (B g B^T gather)",
                        "bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": tf32_peak, "unit": "TFLOP/s",
                        "frac": flops / (ms * 1e-3) / 1e12 / tf32_peak, "traffic": None, "algorithmic_flops": flops,
                        "algorithmic_bytes": bytes_alg, "peak_source": pk["source"] + " bf16 / 2",
                        "kernels_ms": {"conv_bwd": ms_p, "imtrans_bwd": ms_g},
                        "conv_bwd_tflops": flops / (ms_p * 1e-3) / 1e12,
                        "imtrans_bwd_gbs": (64.0 * P * C + 4.0 * B * C * H * W) / (ms_g * 1e-3) / 1e9}}
    del X, V, dYs, hold
    torch.cuda.empty_cache()
    if math == "tf32":     # the vendor library's rate on the two gradient products (dV = dM.W^T, dW = V^T.dM), for scale
        rec["library_tf32"] = library_tf32(ctx, [(16, P, K, C), (16, C, P, K)])
    return rec


def sub_resnet(ctx, args, steps, total=256):
    """configs.cfg4: ResNet-18-var forward, `total` images sharded over the ranks (strong scaling), replayed as a CUDA graph;
    under more than one rank the NCCL all-gather of the logits is timed beside it."""
    import wg2x2
    from resnet18_var import ResNet18Var
    torch = ctx.torch
    lo, hi = wg2x2.shard.shard_range(total, ctx.world, ctx.rank)
    n = hi - lo
    model = ResNet18Var(stage5_pool=not args.stage5_at_14, math=args.math, layout=args.net_layout).to(ctx.dev).eval()
    gen = torch.Generator().manual_seed(100 + ctx.rank)
    imgs_h = torch.randn((n, 3, 224, 224), generator=gen).pin_memory()
    imgs = [imgs_h.to(ctx.dev) + 0.0 * i for i in range(2)]
    with torch.no_grad():
        for i in range(2):
            model(imgs[i % 2])
        torch.cuda.synchronize()
        graphs, outs = None, None
        if not args.no_graph:     # the forward pass is a fixed sequence of ~150 launches: capture it once per input buffer and replay
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graphs, outs = [], []
            with torch.cuda.stream(side):
                for k in range(2):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        outs.append(model(imgs[k]))
                    graphs.append(g)
            torch.cuda.current_stream().wait_stream(side)
        last = {}

        def fwd(i):
            if graphs is not None:
                graphs[i % 2].replay()
                last["y"] = outs[i % 2]
            else:
                last["y"] = model(imgs[i % 2])

        ms = timed(ctx, fwd, steps, warmup=2)
        check_status(wg2x2)
        rec = {"ms_per_step": ms, "steps": steps, "img_s": total / (ms * 1e-3), "scaling": "strong", "total_batch": total, "per_gpu_batch": n,
               "image": 224, "stage5_spatial": 14 if args.stage5_at_14 else 7, "layout": args.net_layout, "dtype": "tf32" if args.math == "tf32" else "f32",
               "launch": "eager" if graphs is None else "one CUDA graph per input buffer, replayed",
               "winograd_tflops_dense": model.winograd_flops(total) / (ms * 1e-3) / 1e12,
               "winograd_layers": "16, densities 0.6/0.4/0.3/0.2 by stage; 7x7 stem + pool1 and the max-pools on this library's kernels; 1x1 shortcuts, FC on stock torch"}
        if ctx.world > 1:      # the one collective of the sharded forward: every rank receives all logits (not on the timed path above)
            gm = timed(ctx, lambda i: wg2x2.shard.gather_batch(last["y"], total), 10, warmup=2)
            full = wg2x2.shard.gather_batch(last["y"], total)
            assert tuple(full.shape) == (total, 1000) and torch.equal(full[lo:hi], last["y"])
            rec["gather_ms"] = gm
            rec["gather"] = "NCCL all_gather of the (%d, 1000) logits shards over NVLink, %d ranks" % (n, ctx.world)
        # end to end: images from pinned host memory, logits back to the host.  Two input buffers (one graph each): the
        # copy of step i+1's images runs on a copy stream under step i's forward pass, as a serving loop would do it
        logits_h = [torch.empty((n, 1000)).pin_memory() for _ in range(2)]
        xd = torch.empty_like(imgs[0])
        copy_stream = torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]
        for ev in ev_free:
            ev.record()

        def e2e(i):
            cur = torch.cuda.current_stream()
            if graphs is not None:      # graph k reads imgs[k] and writes outs[k]
                k = i % 2
                copy_stream.wait_event(ev_free[k])          # the forward pass that last read imgs[k] is done
                with torch.cuda.stream(copy_stream):
                    imgs[k].copy_(imgs_h, non_blocking=True)
                    ev_in[k].record()
                cur.wait_event(ev_in[k])
                graphs[k].replay()
                ev_free[k].record()
                logits_h[k].copy_(outs[k], non_blocking=True)
            else:
                xd.copy_(imgs_h, non_blocking=True)
                logits_h[0].copy_(model(xd), non_blocking=True)

        e2e_ms = timed(ctx, e2e, max(4, min(steps, 8)), warmup=2)
        rec["e2e"] = {"value": total / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": imgs_h.numel() * 4,
                      "d2h_bytes_per_step": logits_h[0].numel() * 4, "ms_per_step": e2e_ms,
                      "pipeline": "two input buffers; the host-to-device copy of a step runs under the previous step's forward pass"
                                  if graphs is not None else "one stream, copies and forward pass in turn"}
    del model, graphs, outs, imgs, last
    torch.cuda.empty_cache()
    return rec


def reference_gpu(ctx, wl):
    """The reference's own forward kernels (oracle/_ref/libwg_ref_cuda.so: its *.cu.cc compiled unmodified for sm_100a) on the
    headline workload: Winograd2x2ImTransComputeLauncher, the ReLU its layer wrapper applies, Winograd2x2ConvComputeLauncher
    (16 cublasSgemmBatched products in FP32 + Output_transform).  NHWC, forward only, even sizes only (the upstream gradient
    kernels read out of bounds on odd sizes and are never run here).  A baseline figure, measured beside this library's."""
    so = os.path.join(ROOT, "oracle", "_ref", "libwg_ref_cuda.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/libwg_ref_cuda.so not built (make -C oracle ref REF=<reference checkout>)"}
    torch = ctx.torch
    B, C, K, H, W = wl["B"], wl["C"], wl["K"], wl["H"], wl["W"]
    if H % 2 or W % 2:
        return {"unavailable": "odd image size"}
    ref = ctypes.CDLL(so)
    Pv = ctypes.c_void_p
    nH, nW = H // 2, W // 2
    Xh, Wth = make_inputs(wl, seed=1)
    xs = [torch.from_numpy(np.ascontiguousarray(np.transpose(Xh, (0, 2, 3, 1)))).to(ctx.dev) + 0.0 * i for i in range(2)]
    wt = torch.from_numpy(Wth).to(ctx.dev)
    V = torch.empty((16, B, nH, nW, C), device=ctx.dev)
    Y = torch.empty((B, H, W, K), device=ctx.dev)
    tmp = torch.empty(16 * B * nH * nW * K, device=ctx.dev)
    ptrs = torch.empty(80, dtype=torch.int64, device=ctx.dev)
    torch.cuda.synchronize()

    def step(i):   # the upstream launchers use the legacy default stream, as does torch here
        ref.wgref_imtrans(Pv(xs[i % 2].data_ptr()), Pv(V.data_ptr()), C, B, H, W)
        torch.relu_(V)
        ref.wgref_conv(Pv(V.data_ptr()), Pv(wt.data_ptr()), Pv(Y.data_ptr()), Pv(tmp.data_ptr()), Pv(ptrs.data_ptr()), C, B, nH, nW, K)

    for i in range(2):
        step(i)
    torch.cuda.synchronize()
    n = 12
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    t0 = time.perf_counter()
    for i in range(n):
        ev[i][0].record()
        step(i)
        ev[i][1].record()
    torch.cuda.synchronize()
    wall_ms = 1e3 * (time.perf_counter() - t0) / n
    dev = sorted(a.elapsed_time(b) for a, b in ev)
    ms = dev[n // 2]
    # every upstream call creates and destroys a cuBLAS handle (host work and a device synchronisation), so the step takes
    # longer on the clock than on the device: both are given
    return {"ms_per_step": ms, "img_s": B / (ms * 1e-3), "kind": "_ref", "layout": "NHWC", "dtype": "f32", "steps": n,
            "ms_per_step_min": dev[0], "wall_ms_per_step": wall_ms,
            "what": "upstream imTrans + ReLU + conv launchers (cublasSgemmBatched FP32, cuBLAS handle created and destroyed per call, as "
                    "upstream); ms_per_step = median device time of a step (CUDA events), wall_ms_per_step = host clock per step"}


# ---------------------------------------------------------------------------------------------------------
# The headline workload
# ---------------------------------------------------------------------------------------------------------
def run_layer(args, ctx):
    import wg2x2  # raises if the CUDA library is missing: there is no fallback
    torch = ctx.torch
    wl = dict(WORKLOADS[args.workload])
    if args.batch > 0:
        wl["B"] = args.batch
    path = "fused" if args.fused else args.path
    L = LayerFwd(ctx, wl, args.layout, args.math, path)
    B, C, K, H, W = wl["B"], wl["C"], wl["K"], wl["H"], wl["W"]

    # ---- the timed region: `steps` launches back to back between two events, nothing else on the stream
    sampler = ClockSampler(ctx.local)
    for i in range(args.warmup):
        L.step(i)
    ctx.barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    t_start.record()
    for i in range(args.steps):
        L.step(i)
    t_end.record()
    torch.cuda.synchronize()
    clocks = sampler.finish(wall0, time.time())
    ctx.barrier()
    ms_step = ctx.max_over_ranks(t_start.elapsed_time(t_end)) / args.steps
    check_status(wg2x2)

    pk = peaks()
    roof, which = L.roofline(pk)
    if L.use_fused:
        # one launch per step: the kernel's average launch duration over the timed region is ms_per_step; the duration of a
        # launch bracketed by its own events (no overlap with its neighbours' launch latency) is kept beside it
        roof["achieved_isolated_launch"], roof["frac_isolated_launch"] = roof["achieved"], roof["frac"]
        roof["achieved"] = roof["algorithmic_bytes"] / (ms_step * 1e-3) / 1e9
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["duration_ms"] = ms_step
    traffic = NCU_TRAFFIC.get((args.workload, B, args.layout, which))
    roof["traffic"], roof["traffic_source"] = (traffic if traffic else (None, None))
    if L.use_fused and ctx.rank == 0 and not args.only_headline:
        # for context: the same layer as two kernels with V through HBM, each with its own HBM roofline fraction
        t1 = timed(Ctx1(ctx), L.imtrans, 50)
        t2 = timed(Ctx1(ctx), L.conv, 50)
        k1_bytes, k2_bytes = L.bytesX + L.bytesV, L.bytesV + L.bytesW + L.bytesY
        roof["two_kernel_path"] = {"imtrans_fwd_ms": t1, "conv_fwd_ms": t2, "imtrans_fwd_frac": k1_bytes / (t1 * 1e-3) / 1e9 / pk["hbm_gbs"],
                                   "conv_fwd_frac": k2_bytes / (t2 * 1e-3) / 1e9 / pk["hbm_gbs"], "layer_ms": t1 + t2,
                                   "note": "the same layer as input transform + product kernels with V through HBM (bench.py --path two-kernel)"}

    out = {
        "metric": METRIC, "value": ctx.world * B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": ctx.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "tf32" if args.math == "tf32" else "f32", "data": "synthetic",
        "config": {"workload": args.workload, "layer": wl, "layout": args.layout, "per_gpu_batch": B,
                   "l2": "%d rotating input buffers (%.0f MB); %.0f MB moved per step" % (L.nbuf, L.nbuf * L.bytesX / 1e6, L.layer_bytes() / 1e6),
                   "weights": "prepared once outside the timed region (wg2x2_weights_prepare)",
                   "timing": "two CUDA events around the steps; per-kernel durations from a separate pass afterwards",
                   "path": "one fused kernel (wg2x2_layer_fwd_prepared's choice for this shape)" if L.use_fused else "two kernels, V through HBM"},
        "layer_gbs": L.layer_bytes() * ctx.world / (ms_step * 1e-3) / 1e9,
        "layer_tflops": L.flops * ctx.world / (ms_step * 1e-3) / 1e12,
        "roofline": roof, "clocks": clocks, "gpu_launches": args.steps * (1 if L.use_fused else 2),
    }

    # ---- end to end through the public call with host buffers
    if not args.only_headline:
        out["e2e"] = run_e2e(args, ctx, L)
        out["config"]["e2e"] = ("wg2x2.HostLayerPipeline.submit: pinned host X -> pinned host Y every step, %d chunks, H2D / kernels / D2H on "
                                "three streams, consecutive steps overlapped (two host output buffers)" % args.e2e_chunks)
    del L
    torch.cuda.empty_cache()

    # ---- the other workloads, each measured in this run (all ranks take part; cfg4 is sharded over them)
    if not args.only_headline and not args.no_configs and args.workload == "cfg2" and args.batch == 0:
        cfgs = {}
        for name, fn in (("cfg1", lambda: sub_layer_fwd(ctx, "cfg1", args, 200)), ("cfg3", lambda: sub_layer_fwd(ctx, "cfg3", args, 60)),
                         ("cfg5", lambda: sub_backward(ctx, args, 30)), ("cfg4", lambda: sub_resnet(ctx, args, 8))):
            try:
                cfgs[name] = fn()
            except Exception as e:     # a failed sub-record must not take the headline with it
                if ctx.world > 1:
                    raise
                cfgs[name] = {"error": "%s: %s" % (type(e).__name__, e)}
        out["configs"] = cfgs
    if ctx.rank == 0 and not args.only_headline:
        if args.workload == "cfg2" and args.batch == 0 and not args.no_ref_gpu:
            try:
                out["reference_gpu"] = reference_gpu(ctx, wl)
            except Exception as e:
                out["reference_gpu"] = {"unavailable": "%s: %s" % (type(e).__name__, e)}
        if not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(wl)
            if "configs" in out and "cfg5" in out["configs"] and "error" not in out["configs"]["cfg5"]:
                out["configs"]["cfg5"]["cpu_baseline"] = cpu_baseline_bwd()
    if ctx.rank == 0:
        print(json.dumps(out))


class Ctx1:
    """A view of a Ctx that times on this rank alone (no barrier, no reduction): for context figures taken by rank 0 only."""

    def __init__(self, ctx):
        self.torch, self.world, self.rank = ctx.torch, 1, ctx.rank

    def barrier(self):
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        return float(ms)


def run_e2e(args, ctx, L):
    """The same layer through wg2x2.HostLayerPipeline.submit: pinned host X -> device -> pinned host Y inside the timed region.
    Beside it, the two copies alone (no kernels), all ranks at once: the host-side ceiling of the box."""
    import wg2x2
    torch = ctx.torch
    wl = L.wl
    node = wg2x2.host.bind_to_gpu_node(ctx.local) if not args.no_numa_bind else None   # before the pinned allocations: first touch
    Xpin = torch.from_numpy(L.Xh).pin_memory()
    Ypins = [torch.empty(L.Y.shape, dtype=torch.float32).pin_memory() for _ in range(2)]
    pipe = wg2x2.HostLayerPipeline(wl["B"], wl["H"], wl["W"], wl["C"], wl["K"], layout=L.layout, math=L.math, relu=True, chunks=args.e2e_chunks)
    e2e_steps = max(3, min(args.steps, 50))
    done = [None]

    def step(i):   # one host output buffer per step in flight: step n+1 is submitted while step n is still being read back
        done[0] = pipe.submit(Xpin, L.Wt, Ypins[i % 2])

    for i in range(2):
        step(i)
    ctx.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(e2e_steps):
        step(i)
    torch.cuda.current_stream().wait_event(done[0])    # the last step's results are in host memory
    b.record()
    ctx.barrier()
    e2e_ms = ctx.max_over_ranks(a.elapsed_time(b)) / e2e_steps
    # the copies alone, both directions at once on two streams
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    xd, yd = torch.empty_like(L.Xs[0]), L.Y
    ctx.barrier()
    n_copy = 5
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    with torch.cuda.stream(s_in):
        ev[0].record()
        for _ in range(n_copy):
            xd.copy_(Xpin, non_blocking=True)
        ev[1].record()
    with torch.cuda.stream(s_out):
        ev[2].record()
        for _ in range(n_copy):
            Ypins[0].copy_(yd, non_blocking=True)
        ev[3].record()
    ctx.barrier()
    h2d = n_copy * L.bytesX / (ev[0].elapsed_time(ev[1]) * 1e-3) / 1e9
    d2h = n_copy * L.bytesY / (ev[2].elapsed_time(ev[3]) * 1e-3) / 1e9
    return {"value": ctx.world * wl["B"] / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": L.bytesX, "d2h_bytes_per_step": L.bytesY,
            "ms_per_step": e2e_ms, "h2d_gbs_per_rank": L.bytesX / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": L.bytesY / (e2e_ms * 1e-3) / 1e9,
            "copies_alone": {"h2d_gbs": -ctx.max_over_ranks(-h2d), "d2h_gbs": -ctx.max_over_ranks(-d2h),
                             "note": "slowest rank's rate with both directions busy on every rank at once and no kernels: the host-side ceiling"},
            "host_binding": node}


def run_single(args, ctx, rec_fn, metric, scaling, launches_per_step):
    """--workload cfg4 / cfg5 on their own: the sub-record promoted to a line of its own."""
    sampler = ClockSampler(ctx.local)
    wall0 = time.time()
    rec = rec_fn()
    clocks = sampler.finish(wall0, time.time())
    if ctx.rank == 0:
        out = {"metric": metric, "value": rec["img_s"], "unit": UNIT, "n_gpus": ctx.world, "steps": rec["steps"], "warmup": 3,
               "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": rec["dtype"],
               "data": "synthetic", "config": dict({"workload": args.workload}, **{k: v for k, v in rec.items() if k not in ("roofline", "e2e")}),
               "clocks": clocks, "gpu_launches": rec["steps"] * launches_per_step}
        for k in ("roofline", "e2e"):
            if k in rec:
                out[k] = rec[k]
        print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--math", default=os.environ.get("WG2X2_BENCH_MATH", "tf32"), choices=["tf32", "fp32"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS) + ["cfg4", "cfg5"])
    ap.add_argument("--bwd-math", default="tf32", choices=["fp32", "tf32"], help="cfg5: math mode of the gradient products")
    ap.add_argument("--stage5-at-14", action="store_true", help="cfg4: leave pool4 out, as the reference script does")
    ap.add_argument("--layout", default="NCHW", choices=["NCHW", "NHWC"])
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch of the workload (profiling on a small case)")
    ap.add_argument("--e2e-chunks", type=int, default=2, help="chunks of the host-buffer pipeline")
    ap.add_argument("--path", default="auto", choices=["auto", "fused", "two-kernel"],
                    help="layer forward: the one-kernel path (X -> Y, V never stored), the two kernels, or (auto) whichever "
                         "wg2x2_layer_fwd_prepared picks for the shape")
    ap.add_argument("--fused", action="store_true", help="same as --path fused")
    ap.add_argument("--net-layout", default="NCHW", choices=["NHWC", "NCHW"],
                    help="cfg4: physical layout of the activations (NCHW: the 56x56 and 28x28 layers run as one kernel each)")
    ap.add_argument("--no-graph", action="store_true", help="cfg4: launch the network eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="leave out the sub-records of the other workloads")
    ap.add_argument("--no-ref-gpu", action="store_true", help="leave out the reference's own CUDA kernels")
    ap.add_argument("--no-numa-bind", action="store_true", help="e2e: do not bind the host thread to the GPU's NUMA node")
    ap.add_argument("--only-headline", action="store_true",
                    help="the timed region and the per-kernel pass only (for profiler captures: few launches, small footprint)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    ctx = Ctx()
    try:
        if args.workload == "cfg4":
            run_single(args, ctx, lambda: sub_resnet(ctx, args, max(3, min(args.steps, 30)), total=args.batch or 256),
                       "resnet18_var_forward_throughput", "strong", 35)
        elif args.workload == "cfg5":
            run_single(args, ctx, lambda: sub_backward(ctx, args, max(3, min(args.steps, 200)), math=args.bwd_math, batch=args.batch),
                       "winograd_relu_conv_layer_bwd_throughput", "weak", 6)
        else:
            run_layer(args, ctx)
    finally:
        ctx.close()


if __name__ == "__main__":
    main()
