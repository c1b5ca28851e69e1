#!/usr/bin/env python
"""Benchmark of the convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = forward + gradInputs + gradWeights of the single ResNet-style 3x3 layer
(float32, N=128 per GPU, C=K=256, 14x14, pad 1, stride 1), 88.8 GFLOP per GPU, on seeded
synthetic tensors.  With N GPUs (one process per GPU, launched by torch.distributed.run)
every rank runs the same layer on its own batch shard and the filter gradient is summed
over ranks with one NCCL all-reduce per step (weak scaling).

Printed JSON (rank 0): `value` is TFLOP/s over all GPUs with the tensors resident in HBM in
the library's channels-last device format, timed per step with CUDA events on the library's
stream, L2 flushed between steps; `e2e` is the same step driven from pinned host arrays in
the reference's NCHW layout, copies and layout conversion included; `roofline` describes the
dominant kernel (implicit-GEMM forward/gradInputs); `cpu_baseline` is the CPU restatement of
the reference's im2col+gemm path timed on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORK = dict(name="resnet3x3_f32_N128_C256_K256_14x14_fwd+gradInputs+gradWeights",
            N=128, C=256, K=256, H=14, W=14, k=3, pad=1)
SEED = 1235


def flops_per_pass(w):
    return 2.0 * w["N"] * w["K"] * w["C"] * w["k"] * w["k"] * w["H"] * w["W"]


def make_inputs(rank):
    w = WORK
    rs = np.random.RandomState(SEED + rank)
    x = rs.standard_normal((w["N"], w["C"], w["H"], w["W"])).astype(np.float32)
    wt = (np.random.RandomState(SEED).standard_normal((w["K"], w["C"], w["k"], w["k"])) *
          np.sqrt(2.0 / (w["C"] * w["k"] * w["k"]))).astype(np.float32)   # same filters on every rank
    dy = rs.standard_normal((w["N"], w["K"], w["H"], w["W"])).astype(np.float32)
    return x, wt, dy


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(bf16=float(p["bf16_tflops"]), bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    hbm=float(p["hbm_gbs"]), source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.th.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_step(O, x, wt, dy, w):
    kw = dict(border_mode=(w["pad"], w["pad"]), filter_flip=True)
    O.conv2d(x, wt, **kw)
    O.conv2d_grad_inputs(wt, dy, (w["H"], w["W"]), **kw)
    O.conv2d_grad_weights(x, dy, (w["k"], w["k"]), **kw)


def time_cpu(steps, warmup):
    """The CPU restatement of the reference path (im2col + BLAS gemm, OpenMP over the batch)."""
    from oracle import corr_oracle as O
    O.set_threads(len(os.sched_getaffinity(0)))      # all host cores, whatever the launcher exported
    x, wt, dy = make_inputs(0)
    for _ in range(warmup):
        cpu_step(O, x, wt, dy, WORK)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(O, x, wt, dy, WORK)
        ts.append(time.perf_counter() - t0)
    ms = 1e3 * float(np.mean(ts))
    return ms, O.threads(), ("OpenBLAS sgemm" if O.lib().blas_path else "portable C gemm")


def time_reference_corrmm(steps, warmup):
    """The reference's own CPU path: CorrMM, CorrMM_gradInputs and CorrMM_gradWeights
    (theano/tensor/nnet/corr.py:592,801,685; generated C around BLAS sgemm, OpenMP over the batch)
    compiled by the reference itself, on the full workload.  Raises when the reference cannot be
    imported or cannot compile here."""
    from oracle import ref_theano
    if not ref_theano.available():
        raise RuntimeError("no reference tree or installed copy")
    theano = ref_theano.import_theano()
    import theano.tensor as T
    from theano.tensor.nnet import corr
    w_ = WORK
    x, wt, dy = make_inputs(0)
    xs, ws, gs = T.ftensor4(), T.ftensor4(), T.ftensor4()
    bm = (w_["pad"], w_["pad"])
    wf = ws[:, :, ::-1, ::-1]                                   # filter_flip=True (nnet/opt.py:84-92)
    y = corr.CorrMM(border_mode=bm)(xs, wf)
    dx = corr.CorrMM_gradInputs(border_mode=bm)(wf, gs, (w_["H"], w_["W"]))
    dw = corr.CorrMM_gradWeights(border_mode=bm)(xs, gs, (w_["k"], w_["k"]))[:, :, ::-1, ::-1]
    f = theano.function([xs, ws, gs], [y, dx, dw])
    ops = [type(n.op).__name__ for n in f.maker.fgraph.toposort()]
    assert "CorrMM" in ops and "CorrMM_gradInputs" in ops and "CorrMM_gradWeights" in ops, ops
    for _ in range(warmup):
        f(x, wt, dy)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        f(x, wt, dy)
        ts.append(time.perf_counter() - t0)
    blas = theano.config.blas.ldflags
    gemm = "OpenBLAS sgemm, openmp=%s" % theano.config.openmp if blas else "NumPy-backed gemm (no BLAS to link), openmp=False"
    cores = int(os.environ.get("OMP_NUM_THREADS", "1")) if theano.config.openmp else 1
    return 1e3 * float(np.mean(ts)), cores, gemm


def run_reference(args, rank):
    if rank != 0:
        return
    kind, note = "reference", None
    try:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))   # whatever the launcher exported
        ms, cores, gemm = time_reference_corrmm(args.steps, max(args.warmup, 1))
        gemm = "reference CorrMM ops, " + gemm
    except Exception as e:  # noqa: BLE001  (reference not importable / not compilable here)
        kind, note = "port", "reference not runnable here (%s: %s); timed its CPU restatement" % (type(e).__name__, str(e)[:120])
        ms, cores, gemm = time_cpu(args.steps, max(args.warmup, 1))
    tf = 3 * flops_per_pass(WORK) / (ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": "conv TFLOP/s (fwd+gradInputs+gradWeights)", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "images_per_s": WORK["N"] / (ms * 1e-3),
        "config": {"workload": WORK["name"], "timing": "wall clock on host cores; inputs larger than the CPU caches"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                         "sample": "full workload (batch 128), %d steps, %s" % (args.steps, gemm)},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if note:
        line["cpu_baseline"]["note"] = note
    print(json.dumps(line))


def run_b200(args, rank, local_rank, world):
    from theano_b200 import shim
    dist = None
    if world > 1:
        import torch.distributed as dist  # rendezvous and host-side reductions only
        dist.init_process_group("gloo")
    # The all-reduce of 2.4 MB runs beside two convolution kernels that leave 20 SMs free: measured
    # on 8 GPUs, the step shrinks with the number of CTAs NCCL may use (0.448 / 0.319 / 0.253 /
    # 0.225 ms with 2 / 4 / 8 / 16); 16 still fit beside the 128 convolution CTAs.
    os.environ.setdefault("NCCL_MAX_CTAS", "16")
    ctx = shim.Context(local_rank)
    if args.no_autotune:
        ctx.set_autotune(False)
    if world > 1:
        box = [ctx.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx.nccl_init(world, rank, box[0])

    w = WORK
    x, wt, dy = make_inputs(rank)
    kw = dict(border_mode=(w["pad"], w["pad"]), filter_flip=True)
    T = shim.DeviceTensor
    X, DY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, dy, "nhwc")
    Wd = T.from_host(ctx, wt)
    Y = T(ctx, (w["N"], w["K"], w["H"], w["W"]), np.float32, "nhwc")
    DX = T(ctx, x.shape, np.float32, "nhwc")
    DW = T(ctx, wt.shape, np.float32, "nchw")

    def part1():
        shim.device_grad_weights(X, DY, (w["k"], w["k"]), out=DW, **kw)

    def part2():
        shim.device_conv2d(X, Wd, out=Y, **kw)
        shim.device_grad_inputs(Wd, DY, (w["H"], w["W"]), out=DX, **kw)

    # The three calls are recorded once as CUDA graphs and replayed: one driver launch per part
    # instead of the Python and launch overhead of every kernel.  The three passes of one layer
    # do not depend on each other; gradWeights is issued first so that its all-reduce (between
    # the two graphs, on a second stream) runs beside the other two passes, the way the
    # all-reduce of a layer's filter gradient runs beside the rest of a network's backward pass.
    part1(); part2(); ctx.sync()
    if args.no_graph:
        g1 = g2 = None
    else:
        g1, g2 = ctx.capture(part1), ctx.capture(part2)

    def step():
        g1.launch() if g1 else part1()
        if world > 1 and not args.no_collective:
            ctx.allreduce_sum_async(DW.ptr, int(np.prod(wt.shape)), np.float32)
        g2.launch() if g2 else part2()
        if world > 1 and not args.no_collective:
            ctx.comm_wait()

    # clock samples are taken every 100 ms: keep the GPU under this load for about a second
    # before the timed steps so that the record shows the clocks the steps ran at
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    n_warm = max(args.warmup, 3) + args.clock_warm   # the same count on every rank (each step has a collective)
    for i in range(n_warm):
        step()
        if i % 50 == 49:
            ctx.sync()
    ctx.barrier()
    launches0 = ctx.launches
    times = []
    for _ in range(args.steps):
        ctx.flush_l2()
        ctx.barrier()           # all ranks start the step together (also drains the flush)
        ctx.timer_start()
        step()
        times.append(ctx.timer_stop())
    launches = ctx.launches - launches0
    # per-kernel durations: the same calls issued eagerly with an event pair around every launch
    # (on the library's stream), L2 flushed before each step as above
    ctx.kernel_timing(True)
    for _ in range(args.steps):
        ctx.flush_l2()
        part1(); part2()
    conv_ms, conv_n = ctx.kernel_time("conv_umma")
    wg_ms, wg_n = ctx.kernel_time("wgrad_umma")
    ctx.kernel_timing(False)
    clocks = sampler.stop() if rank == 0 else None
    times = np.asarray(times, np.float64)
    if world > 1:
        import torch
        t = torch.from_numpy(times.copy())
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = t.numpy()
    ms = float(times.mean())

    # ---- end to end: pinned host NCHW arrays in, NCHW arrays out, every step -----------------
    xh, wh, dyh = (ctx.pinned_empty(a.shape, np.float32) for a in (x, wt, dy))
    xh[...], wh[...], dyh[...] = x, wt, dy
    yh, dxh, dwh = (ctx.pinned_empty(s, np.float32) for s in (Y.shape, x.shape, wt.shape))
    Xn, DYn, Yn, DXn = (T(ctx, s, np.float32, "nchw") for s in (x.shape, dy.shape, Y.shape, x.shape))

    # PCIe carries both directions at once: uploads run on a background stream, downloads on
    # another, and the batch travels in parts so that the first results go back while the rest
    # still arrives.  dy and the filters go first (gradInputs needs only them), then x (forward);
    # gradWeights needs both whole tensors and comes last.
    nparts = max(1, args.e2e_parts)
    cuts = [w["N"] * i // nparts for i in range(nparts + 1)]
    parts = list(zip(cuts[:-1], cuts[1:]))

    def e2e_step():
        ctx.h2d_bg(DYn.images(*parts[0]).ptr, dyh[parts[0][0]:parts[0][1]])
        ctx.h2d_bg(Wd.ptr, wh)
        for k, (a, b) in enumerate(parts):                        # gradInputs, part by part
            ctx.join_uploads()
            if k + 1 < len(parts):
                ctx.h2d_bg(DYn.images(*parts[k + 1]).ptr, dyh[parts[k + 1][0]:parts[k + 1][1]])
            else:
                ctx.h2d_bg(Xn.images(*parts[0]).ptr, xh[parts[0][0]:parts[0][1]])
            ctx.nchw_to_nhwc(DYn.images(a, b).ptr, DY.images(a, b).ptr, b - a, *dy.shape[1:], np.float32)
            shim.device_grad_inputs(Wd, DY.images(a, b), (w["H"], w["W"]), out=DXn.images(a, b), **kw)
            ctx.d2h_bg(dxh[a:b], DXn.images(a, b).ptr)
        for k, (a, b) in enumerate(parts):                        # forward, part by part
            ctx.join_uploads()
            if k + 1 < len(parts):
                ctx.h2d_bg(Xn.images(*parts[k + 1]).ptr, xh[parts[k + 1][0]:parts[k + 1][1]])
            ctx.nchw_to_nhwc(Xn.images(a, b).ptr, X.images(a, b).ptr, b - a, *x.shape[1:], np.float32)
            shim.device_conv2d(X.images(a, b), Wd, out=Yn.images(a, b), **kw)
            ctx.d2h_bg(yh[a:b], Yn.images(a, b).ptr)
        shim.device_grad_weights(X, DY, (w["k"], w["k"]), out=DW, **kw)
        if world > 1 and not args.no_collective:
            ctx.allreduce_sum_async(DW.ptr, int(np.prod(wt.shape)), np.float32)
            ctx.comm_wait()
        ctx.d2h_bg(dwh, DW.ptr)
        ctx.sync()

    for _ in range(2):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_t = []
    for _ in range(e2e_steps):
        ctx.barrier()
        t0 = time.perf_counter()
        e2e_step()
        e2e_t.append(time.perf_counter() - t0)
    e2e_t = np.asarray(e2e_t, np.float64)
    if world > 1:
        import torch
        t = torch.from_numpy(e2e_t.copy())
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_t = t.numpy()
    e2e_ms = 1e3 * float(e2e_t.mean())
    h2d = xh.nbytes + wh.nbytes + dyh.nbytes
    d2h = yh.nbytes + dxh.nbytes + dwh.nbytes

    if rank != 0:
        if world > 1:
            dist.barrier()
        return
    fl = flops_per_pass(w)
    pk = peaks()
    tf32_peak = pk["bf16"] / 2.0   # kind::tf32 runs at half the 16-bit rate
    conv_avg_ms = conv_ms / max(conv_n, 1)
    achieved = fl / (conv_avg_ms * 1e-3) / 1e12 if conv_n else None
    cpu = None
    if world == 1:
        cms, cores, gemm = time_cpu(5, 1)
        cpu = {"value": 3 * fl / (cms * 1e-3) / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": "full workload (batch 128), 5 steps after 1 warm-up, %s, %.1f ms/step" % (gemm, cms)}
    line = {
        "metric": "conv TFLOP/s (fwd+gradInputs+gradWeights)", "value": 3 * fl * world / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
        "images_per_s": w["N"] * world / (ms * 1e-3),
        "frac_of_tf32_peak": 3 * fl / (ms * 1e-3) / 1e12 / tf32_peak,
        "config": {"workload": w["name"], "per_gpu_batch": w["N"], "parallelism": "dp%d" % world,
                   "collective": ("LEFT OUT (--no-collective, diagnosis)" if args.no_collective else
                                  "ncclAllReduce(sum) of gradWeights on a second stream, beside forward and gradInputs") if world > 1 else "none",
                   "order": "gradWeights, forward, gradInputs",
                   "resident_layout": "channels-last activations (library device format), OIHW filters",
                   "l2": "flushed by a 256 MB write before every timed step", "seed": SEED,
                   "clock_warm_steps": args.clock_warm,   # untimed steps before the warm-up that bring the clocks up
                   "launch": "eager" if args.no_graph else "CUDA graph replay (2 graphs per step)"},
        "clocks": clocks,
        "e2e": {"value": 3 * fl * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "path": "pinned host NCHW -> H2D -> channels-last conversion -> kernels -> D2H; the batch travels in %d parts, uploads and downloads on background streams beside the kernels; wall clock" % nparts},
        "gpu_launches": int(launches),
        "roofline": {"kernel": "conv_slab_kernel<tf32,256> (forward and gradInputs launches)", "bound": "tensor",
                     "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                     "frac": achieved / tf32_peak if achieved else None,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch on this workload
                     # (profiles/conv_slab_tf32_resnet3x3_N128.md): the algorithmic reads; the
                     # 25.7 MB result is still in L2 when the kernel ends
                     "traffic": 28.09e6 + 0.07e6,
                     "flops_per_launch": fl,
                     "peak_source": "%s bf16 burst %.1f / 2 (tf32 = half the 16-bit rate)" % (pk["source"], pk["bf16"]),
                     "launches_timed": conv_n, "avg_launch_ms": conv_avg_ms,
                     "wgrad_umma_avg_ms": wg_ms / max(wg_n, 1)},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))
    if world > 1:
        dist.barrier()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="issue every call eagerly (no CUDA graph replay)")
    ap.add_argument("--e2e-parts", type=int, default=2,
                    help="parts the batch is cut into for the pipelined end-to-end leg")
    ap.add_argument("--no-autotune", action="store_true",
                    help="no timing-based choice between kernel variants (for runs under a profiler, "
                         "whose replays distort the timings): the static preference order is used")
    ap.add_argument("--no-collective", action="store_true",
                    help="diagnosis only: leave out the all-reduce (the printed line is then not a valid result)")
    ap.add_argument("--clock-warm", type=int, default=4000,
                    help="extra untimed steps that keep the GPU loaded while clocks are sampled "
                         "(0 for runs under a profiler)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
