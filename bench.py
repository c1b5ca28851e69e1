#!/usr/bin/env python
"""Benchmark of the convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = forward + gradInputs + gradWeights of all 53 convolutions of ResNet-50 (standard
bottleneck shapes, 7x7 stride-2 stem, stride 2 on the 3x3 of the down-sampling bottlenecks) in
float16 with float32 accumulation, 224 x 224 input, batch 256 per GPU: 6.28 TFLOP per GPU and
step.  Every layer works on its own seeded synthetic tensors of the right shape (a layer-isolated
benchmark: the network's name only supplies the layer shapes).  With N GPUs (one process per
GPU, launched by torch.distributed.run) every rank runs the same layers on its own batch shard
and the filter gradients are summed over ranks: they are written into flat buckets of at least
8 MB in backward order, and each bucket is all-reduced by NCCL on a second stream as soon as its
last layer has been enqueued, beside the rest of the backward pass (weak scaling).

Printed JSON (rank 0): `value` is TFLOP/s over all GPUs with the tensors resident in HBM in the
library's channels-last format, timed per step with CUDA events on the library's stream;
`images_per_s` the same as images; `e2e` is the same step driven from pinned host arrays in the
reference's NCHW layout, copies and layout conversion included; `roofline` describes the
(kernel, layer shape) pair with the largest share of the step and `roofline_step` the whole step
against the sum of its layers' rooflines; `parity` compares results of the timed tensors with
the CPU oracle outside the timed region; `cpu_baseline` is the CPU restatement of the
reference's im2col + gemm path timed on the host cores on a reduced batch.
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

from theano_b200 import workloads as WL  # noqa: E402

BATCH = 256                      # per GPU
SEED = 1238                      # base seed 1234 + config index
DTYPE = np.float16
WORKLOAD = "resnet50_53convs_f16_N256_224x224_fwd+gradInputs+gradWeights"
METRIC = "conv TFLOP/s (fwd+gradInputs+gradWeights)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(f16=float(p["bf16_tflops"]), f16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    hbm=float(p["hbm_gbs"]), source="measured")
    return dict(f16=1590.0, f16_sustained=1400.0, hbm=6650.0, source="fallback")


def step_flops(batch):
    return 3.0 * sum(WL.flops(l, batch) for l in WL.resnet50_network())


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


# ======================================================================================
# CPU arms
# ======================================================================================
def cpu_sample_batch(cores):
    """The reference parallelises over the batch only (corr_gemm.c:304): a sample needs at least
    one image per core; CorrMM's time is linear in the batch."""
    return int(min(BATCH, max(16, cores)))


def host_layer_tensors(lay, idx, batch, dtype, rank=0):
    """x and dy differ per rank (its batch shard), the filters are the same on every rank."""
    xs, ws, ys = WL.shapes(lay, batch)
    x = WL.random_tensor(SEED + 1000 * idx + 17 * rank, xs, dtype)
    w = WL.random_tensor(SEED + 1000 * idx + 500, ws, dtype, np.sqrt(2.0 / (lay["C"] * lay["k"] * lay["k"])))
    dy = WL.random_tensor(SEED + 1000 * idx + 700 + 17 * rank, ys, dtype, 0.1)
    return x, w, dy


def time_cpu_port(steps, warmup, batch):
    """The CPU restatement of the reference path (im2col + BLAS gemm, OpenMP over the batch) on the
    53 layers at a reduced batch, float32 (the reference has no float16 CPU path)."""
    from oracle import corr_oracle as O
    cores = len(os.sched_getaffinity(0))
    O.set_threads(cores)
    data = []
    for i, lay in enumerate(WL.RESNET50):
        x, w, dy = host_layer_tensors(lay, i, batch, np.float32)
        data.append((lay, x, w, dy))

    def step():
        for lay, x, w, dy in data:
            kw = WL.conv_kwargs(lay)
            for _ in range(lay["n"]):
                O.conv2d(x, w, **kw)
                O.conv2d_grad_inputs(w, dy, (lay["H"], lay["H"]), **kw)
                O.conv2d_grad_weights(x, dy, (lay["k"], lay["k"]), **kw)
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    return 1e3 * float(np.mean(ts)), O.threads(), ("OpenBLAS sgemm" if O.lib().blas_path else "portable C gemm")


def time_reference_corrmm(steps, warmup, batch):
    """The reference's own CPU path: CorrMM, CorrMM_gradInputs and CorrMM_gradWeights
    (theano/tensor/nnet/corr.py:592,801,685; generated C around BLAS sgemm, OpenMP over the batch)
    compiled by the reference itself, on the 53 layers at a reduced batch in float32.  Raises when
    the reference cannot be imported or cannot compile here."""
    from oracle import ref_theano
    if not ref_theano.available():
        raise RuntimeError("no reference tree or installed copy")
    theano = ref_theano.import_theano()
    import theano.tensor as T
    from theano.tensor.nnet import corr
    fns = []
    for i, lay in enumerate(WL.RESNET50):
        x, w, dy = host_layer_tensors(lay, i, batch, np.float32)
        xs, ws, gs = T.ftensor4(), T.ftensor4(), T.ftensor4()
        kw = dict(border_mode=(lay["p"], lay["p"]), subsample=(lay["s"], lay["s"]))
        wf = ws[:, :, ::-1, ::-1]                                   # filter_flip=True (nnet/opt.py:84-92)
        y = corr.CorrMM(**kw)(xs, wf)
        dx = corr.CorrMM_gradInputs(**kw)(wf, gs, (lay["H"], lay["H"]))
        dw = corr.CorrMM_gradWeights(**kw)(xs, gs, (lay["k"], lay["k"]))[:, :, ::-1, ::-1]
        f = theano.function([xs, ws, gs], [y, dx, dw])
        ops = [type(n.op).__name__ for n in f.maker.fgraph.toposort()]
        assert "CorrMM" in ops and "CorrMM_gradInputs" in ops and "CorrMM_gradWeights" in ops, ops
        fns.append((lay["n"], f, x, w, dy))

    def step():
        for n, f, x, w, dy in fns:
            for _ in range(n):
                f(x, w, dy)
    for _ in range(warmup):
        step()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    blas = theano.config.blas.ldflags
    gemm = "OpenBLAS sgemm, openmp=%s" % theano.config.openmp if blas else "NumPy-backed gemm (no BLAS to link), openmp=False"
    cores = int(os.environ.get("OMP_NUM_THREADS", "1")) if theano.config.openmp else 1
    return 1e3 * float(np.mean(ts)), cores, gemm


def run_reference(args, rank):
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    batch = cpu_sample_batch(cores)
    kind, note = "reference", None
    try:
        os.environ["OMP_NUM_THREADS"] = str(cores)                  # whatever the launcher exported
        ms, used, gemm = time_reference_corrmm(args.steps, max(args.warmup, 1), batch)
        gemm = "reference CorrMM ops, " + gemm
    except Exception as e:  # noqa: BLE001  (reference not importable / not compilable here)
        kind, note = "port", "reference not runnable here (%s: %s); timed its CPU restatement" % (type(e).__name__, str(e)[:120])
        ms, used, gemm = time_cpu_port(args.steps, max(args.warmup, 1), batch)
    tf = step_flops(batch) / (ms * 1e-3) / 1e12
    sample = ("the 53 layers at batch %d instead of %d, float32 (CorrMM is linear in the batch, corr_gemm.c:304), "
              "%d steps, %s" % (batch, BATCH, args.steps, gemm))
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms * BATCH / batch,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "images_per_s": batch / (ms * 1e-3),
        "config": {"workload": WORKLOAD, "per_gpu_batch": BATCH, "sample_batch": batch,
                   "timing": "wall clock on host cores; ms_per_step scaled to batch %d" % BATCH},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": used, "kind": kind, "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if note:
        line["cpu_baseline"]["note"] = note
    print(json.dumps(line))


# ======================================================================================
# the B200 arm
# ======================================================================================
class Net(object):
    """The 53 layers with their device tensors: per layer instance its own channels-last x, y, dy,
    dx (22 GB at batch 256) and its filters; filter gradients live in the buckets."""

    def __init__(self, ctx, shim, dp, rank, world, batch, dw_dtype, bucket_bytes):
        self.ctx, self.shim, self.batch = ctx, shim, batch
        self.layers = WL.resnet50_network()
        T = shim.DeviceTensor
        names = [WL.layer_name(l) for l in WL.RESNET50]
        self.host = {}                                     # distinct shape -> (x, w, dy) host arrays
        self.idx = [names.index(WL.layer_name(l)) for l in self.layers]
        self.X, self.W, self.DY, self.Y, self.DX = [], [], [], [], []
        for lay, k in zip(self.layers, self.idx):
            if k not in self.host:
                self.host[k] = host_layer_tensors(lay, k, batch, DTYPE, rank)
            x, w, dy = self.host[k]
            self.X.append(T.from_host(ctx, x, "nhwc"))
            self.W.append(T.from_host(ctx, w))
            self.DY.append(T.from_host(ctx, dy, "nhwc"))
            self.Y.append(T(ctx, dy.shape, DTYPE, "nhwc"))
            self.DX.append(T(ctx, x.shape, DTYPE, "nhwc"))
        # gradients become ready in backward order: the last layer first
        self.order = list(range(len(self.layers) - 1, -1, -1))
        elems = [int(np.prod(self.W[i].shape)) for i in self.order]
        self.buckets = dp.GradBuckets(ctx, elems, dw_dtype, bucket_bytes, world)
        self.DW = [None] * len(self.layers)
        for j, i in enumerate(self.order):
            self.DW[i] = T(ctx, self.W[i].shape, dw_dtype, "nchw", _ptr=self.buckets.ptr(j))
        self.descs = [shim.layer_desc(self.X[i].shape, self.W[i].shape, dtype=DTYPE, **WL.conv_kwargs(l))
                      for i, l in enumerate(self.layers)]

    def prepack(self):
        """The packed forms of all filter banks for forward and gradInputs, one launch: what a
        training step does once after the optimizer has written new filters."""
        self.ctx.prepack(self.descs, [w.ptr for w in self.W])

    def fwd(self, i):
        lay = self.layers[i]
        self.shim.device_conv2d(self.X[i], self.W[i], out=self.Y[i], **WL.conv_kwargs(lay))

    def dgrad(self, i):
        lay = self.layers[i]
        self.shim.device_grad_inputs(self.W[i], self.DY[i], (lay["H"], lay["H"]), out=self.DX[i], **WL.conv_kwargs(lay))

    def wgrad(self, i):
        lay = self.layers[i]
        self.shim.device_grad_weights(self.X[i], self.DY[i], (lay["k"], lay["k"]), out=self.DW[i], **WL.conv_kwargs(lay))

    def forward_pass(self):
        self.prepack()
        for i in range(len(self.layers)):
            self.fwd(i)

    def backward_segments(self):
        """The backward pass cut where a bucket completes: [(layer indices, bucket position j)]."""
        segs, cur = [], []
        for j, i in enumerate(self.order):
            cur.append(i)
            if j in self.buckets._bucket_of_last:
                segs.append((cur, j))
                cur = []
        assert not cur
        return segs


def run_b200(args, rank, local_rank, world):
    from theano_b200 import dp, shim
    dist = None
    if world > 1:
        import torch.distributed as dist  # rendezvous and host-side reductions only
        dist.init_process_group("gloo")
    # NCCL's kernels share the GPU with persistent convolution kernels that fill every SM they run
    # on: NCCL gets a few CTAs (94 MB of gradients per ~12 ms step need little bandwidth) and the
    # convolution kernels leave that many SMs free (a default the environment can override)
    if args.comm_sms > 0:
        os.environ.setdefault("NCCL_MAX_CTAS", str(args.comm_sms))
    ctx = shim.Context(local_rank)
    if world > 1 and not args.no_collective and args.comm_sms > 0:
        ctx.set_sm_count(148 - args.comm_sms)
    if args.no_autotune:
        ctx.set_autotune(False)
    if world > 1:
        box = [ctx.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx.nccl_init(world, rank, box[0])
    dw_dtype = np.float32 if args.dw_dtype == "f32" else np.float16
    net = Net(ctx, shim, dp, rank, world, BATCH, dw_dtype, args.bucket_mb << 20)
    nl = len(net.layers)
    segs = net.backward_segments()
    collective = world > 1 and not args.no_collective

    def bwd_segment(layers):
        for i in layers:
            net.wgrad(i)
            net.dgrad(i)

    # One eager pass (kernel choice by timing, memory pool warm), then everything is recorded as
    # CUDA graphs: the forward pass as one graph, the backward pass as one graph per bucket, with
    # the bucket's all-reduce issued between the graphs on the communication stream.
    net.forward_pass()
    for layers, _ in segs:
        bwd_segment(layers)
    ctx.sync()
    if args.no_graph:
        g_fwd, g_bwd = None, [None] * len(segs)
    else:
        g_fwd = ctx.capture(net.forward_pass)
        g_bwd = [ctx.capture(lambda layers=layers: bwd_segment(layers)) for layers, _ in segs]

    def step():
        g_fwd.launch() if g_fwd else net.forward_pass()
        for (layers, j), g in zip(segs, g_bwd):
            g.launch() if g else bwd_segment(layers)
            if collective:
                net.buckets.ready(j)
        if collective:
            net.buckets.wait()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    n_warm = max(args.warmup, 3) + args.clock_warm   # the same count on every rank (each step has collectives)
    for i in range(n_warm):
        step()
        if i % 10 == 9:
            ctx.sync()
    ctx.barrier()
    launches0 = ctx.launches
    times = []
    for _ in range(args.steps):
        ctx.barrier()           # all ranks start the step together
        ctx.timer_start()
        step()
        times.append(ctx.timer_stop())
    launches = ctx.launches - launches0
    clocks = sampler.stop() if rank == 0 else None
    times = np.asarray(times, np.float64)
    if world > 1:
        import torch
        t = torch.from_numpy(times.copy())
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = t.numpy()
    ms = float(times.mean())

    # ---- per-kernel durations: every call issued eagerly with an event pair around every launch of
    # the library's kernels (on its stream), layer by layer -------------------------------------
    fams = ("conv_umma", "wgrad_umma", "wgrad_reduce", "pack", "transpose", "direct")
    per_call = []                                    # (layer index, direction, {family: (ms, launches)})
    prepack_ms = (0.0, 0)
    if rank == 0:
        ctx.kernel_timing(True)
        net.prepack()
        prepack_ms = ctx.kernel_time("pack")
        ctx.kernel_timing(False)
        for i in range(nl):
            for name, call in (("fwd", net.fwd), ("dgrad", net.dgrad), ("wgrad", net.wgrad)):
                best = None
                for _ in range(2):                   # the second measurement (steady clocks, warm instruction cache)
                    ctx.kernel_timing(True)
                    call(i)
                    best = {f: ctx.kernel_time(f) for f in fams}
                    ctx.kernel_timing(False)
                per_call.append((i, name, best))

    # ---- parity of the timed tensors against the CPU oracle, outside the timed region ------------
    parity = None
    if rank == 0 or world > 1:
        parity = check_parity(ctx, net, rank, world, dist, collective, step)

    # ---- end to end: pinned host NCHW arrays in, NCHW arrays out, every step ---------------------
    e2e = None if args.no_e2e else run_e2e(ctx, shim, net, rank, world, dist, collective, args)

    if rank != 0:
        if world > 1:
            dist.barrier()
        return
    fl = step_flops(BATCH)
    pk = peaks()
    if args.dump_layers:
        with open(args.dump_layers, "w") as f:
            for i, name, t in per_call:
                lay = net.layers[i]
                rl = max(WL.flops(lay, BATCH) / (pk["f16"] * 1e12), WL.algorithmic_bytes(lay, BATCH, 2) / (pk["hbm"] * 1e9)) * 1e3
                f.write(json.dumps({"i": i, "layer": WL.layer_name(lay), "dir": name, "roofline_ms": rl,
                                    "ms": {k: v[0] for k, v in t.items() if v[1]}}) + "\n")
    fam_ms = {f: sum(c[2][f][0] for c in per_call) for f in fams}
    fam_n = {f: sum(c[2][f][1] for c in per_call) for f in fams}
    fam_ms["pack"] += prepack_ms[0]                  # the one launch that packs every layer's filters
    fam_n["pack"] += prepack_ms[1]
    eager_total = sum(fam_ms.values())
    # the (main kernel, layer shape, direction) with the largest share of the step, with its roofline
    by_shape = {}
    for i, name, t in per_call:
        fam = "wgrad_umma" if name == "wgrad" else "conv_umma"
        key = (net.idx[i], name)
        e = by_shape.setdefault(key, [0.0, 0, fam, i])
        e[0] += t[fam][0]
        e[1] += t[fam][1]
    # the kernel family with the largest share of the step, on the layer shape it spends most time on
    top_fam = "conv_umma" if fam_ms["conv_umma"] >= fam_ms["wgrad_umma"] else "wgrad_umma"
    (kidx, kdir), (kms, kn, kfam, ki) = max(((k, v) for k, v in by_shape.items() if v[2] == top_fam),
                                            key=lambda kv: kv[1][0])
    klay = net.layers[ki]
    k_fl, k_by = WL.flops(klay, BATCH), WL.algorithmic_bytes(klay, BATCH, 2)
    k_avg = kms / max(kn, 1)
    tensor_bound = k_fl / (pk["f16"] * 1e12) >= k_by / (pk["hbm"] * 1e9)
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
    if os.path.exists(tpath):
        traffic = json.load(open(tpath)).get("%s %s" % (WL.layer_name(klay), kdir), {}).get("dram_bytes_per_launch")
    if tensor_bound:
        ach = k_fl / (k_avg * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": pk["f16"], "unit": "TFLOP/s", "frac": ach / pk["f16"]}
    else:
        ach = k_by / (k_avg * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm"], "unit": "GB/s", "frac": ach / pk["hbm"]}
    roof.update({"kernel": "%s kernels (%.0f %% of the step's kernel time), on the layer they spend most time on: %s, %s, batch %d "
                           "(%d launches per step)" % (
                     "gradWeights" if kfam == "wgrad_umma" else "implicit-GEMM convolution (forward and gradInputs)",
                     100.0 * fam_ms[top_fam] / eager_total, WL.layer_name(klay), kdir, BATCH, kn),
                 "traffic": traffic, "avg_launch_ms": k_avg, "share_of_step": kms / eager_total,
                 "flops_per_launch": k_fl, "algorithmic_bytes_per_launch": k_by,
                 "peak_source": "%s (MEASURED_PEAKS.json: bf16 burst = float16 rate, HBM copy)" % pk["source"]})
    # the whole step against the sum of its layers' rooflines max(FLOP / peak, bytes / bandwidth)
    bound_ms = 0.0
    for lay in net.layers:
        bound_ms += 3.0 * max(WL.flops(lay, BATCH) / (pk["f16"] * 1e12), WL.algorithmic_bytes(lay, BATCH, 2) / (pk["hbm"] * 1e9)) * 1e3
    cpu = None
    if world == 1 and not args.no_cpu:
        cb = cpu_sample_batch(len(os.sched_getaffinity(0)))
        cms, cores, gemm = time_cpu_port(3, 1, cb)
        cpu = {"value": step_flops(cb) / (cms * 1e-3) / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "images_per_s": cb / (cms * 1e-3),
               "sample": "the 53 layers at batch %d instead of %d, float32, 3 steps after 1 warm-up, %s, %.0f ms/step "
                         "(time is linear in the batch, corr_gemm.c:304)" % (cb, BATCH, gemm, cms)}
    others = None
    if world == 1 and not args.no_others:
        others = other_configs(ctx, shim, pk)
    e2e_theano = run_e2e_theano(net) if world == 1 and not args.no_e2e else None
    line = {
        "metric": METRIC, "value": fl * world / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "images_per_s": BATCH * world / (ms * 1e-3),
        "frac_of_f16_peak": fl / (ms * 1e-3) / 1e12 / pk["f16"],
        "frac_of_f16_peak_sustained": fl / (ms * 1e-3) / 1e12 / pk["f16_sustained"],
        "config": {"workload": WORKLOAD, "per_gpu_batch": BATCH, "parallelism": "dp%d" % world,
                   "layers": "53 convolutions, stride 2 on the 3x3 of the down-sampling bottlenecks, 8.17 GFLOP forward per image",
                   "collective": ("LEFT OUT (--no-collective, diagnosis)" if args.no_collective else
                                  "ncclAllReduce(sum) per gradient bucket (>= %d MB, %s, %d buckets) on a second stream beside the backward pass; "
                                  "NCCL on %d CTAs, convolution kernels on %d SMs"
                                  % (args.bucket_mb, args.dw_dtype, len(net.buckets.buckets), args.comm_sms, 148 - args.comm_sms)) if world > 1 else "none",
                   "order": "filter packing of all layers (one launch), forward of all layers, then per layer from the last: gradWeights, gradInputs",
                   "resident_layout": "channels-last activations (library device format), OIHW filters",
                   "l2": "no flush: a step touches 22 GB of activations, each tensor once per pass (inputs larger than L2)",
                   "seed": SEED, "sigma_dy": 0.1, "clock_warm_steps": args.clock_warm,
                   "launch": "eager" if args.no_graph else "CUDA graph replay (1 forward graph + %d backward graphs per step)" % len(segs)},
        "clocks": clocks,
        "e2e": e2e,
        "e2e_theano": e2e_theano,
        "gpu_launches": int(launches),
        "roofline": roof,
        "roofline_step": {"sum_of_layer_rooflines_ms": bound_ms, "frac": bound_ms / ms,
                          "note": "sum over layers and passes of max(FLOP / f16 peak, (|X|+|W|+|Y|) bytes / HBM bandwidth)"},
        "kernel_shares": {f: {"ms": fam_ms[f], "launches": fam_n[f], "share": fam_ms[f] / eager_total} for f in fams if fam_n[f]},
        "parity": parity,
        "cpu_baseline": cpu,
        "other_configs": others,
    }
    print(json.dumps(line))
    if world > 1:
        dist.barrier()


def check_parity(ctx, net, rank, world, dist, collective, step):
    """Results of the timed tensors against the CPU oracle (float32 on the float16-rounded inputs).
    Forward and gradInputs on two images of three layers; gradWeights (after the all-reduce when
    there are several ranks: the sum over every rank's shard, corr_gemm.c:443-455 over GPUs) on the
    whole batch of three layers.  Error: max|a - b| / max|b|, tolerance 2e-2."""
    from oracle import corr_oracle as O
    step()
    ctx.sync()
    nl = len(net.layers)
    picks = [nl - 1, nl - 3, 32]           # 512->2048 1x1 @7, 512->512 3x3 @7, a 14x14 layer
    res = {"tolerance": 2e-2, "checks": {}}
    worst = 0.0
    for i in picks:
        lay = net.layers[i]
        kw = WL.conv_kwargs(lay)
        k = net.idx[i]
        x, w, dy = net.host[k]
        wf = w.astype(np.float32)
        if rank == 0:
            for img in (0, net.batch - 1):
                got = net.Y[i].images(img, img + 1).to_host().astype(np.float32)
                e = O.rel_err(got, O.conv2d(x[img:img + 1].astype(np.float32), wf, **kw))
                got = net.DX[i].images(img, img + 1).to_host().astype(np.float32)
                e2 = O.rel_err(got, O.conv2d_grad_inputs(wf, dy[img:img + 1].astype(np.float32), (lay["H"], lay["H"]), **kw))
                res["checks"]["%s fwd[%d]" % (WL.layer_name(lay), img)] = e
                res["checks"]["%s gradInputs[%d]" % (WL.layer_name(lay), img)] = e2
                worst = max(worst, e, e2)
            # gradWeights of the whole job: every rank's shard regenerated from its seed
            want = None
            for r in range(world if collective else 1):
                xr, _, dyr = (x, None, dy) if r == 0 else host_layer_tensors(lay, k, net.batch, DTYPE, r)
                g = O.conv2d_grad_weights(xr.astype(np.float32), dyr.astype(np.float32), (lay["k"], lay["k"]), **kw)
                want = g if want is None else want + g
            j = net.order.index(i)
            got = net.buckets.to_host(j).astype(np.float32).reshape(want.shape)
            e = O.rel_err(got, want)
            res["checks"]["%s gradWeights%s" % (WL.layer_name(lay), " summed over %d ranks" % world if collective else "")] = e
            worst = max(worst, e)
    if world > 1:
        dist.barrier()
    if rank != 0:
        return None
    res["max_rel_err"] = worst
    res["ok"] = bool(worst < res["tolerance"])
    return res


def run_e2e(ctx, shim, net, rank, world, dist, collective, args):
    """The same step from pinned host arrays in the reference's NCHW layout: per layer x, w and dy
    are uploaded, converted to channels-last on the device, the three passes run, y and dx are
    converted back and y, dx and dw downloaded.  Uploads and downloads run on two background
    streams beside the kernels (PCIe moves both ways at once)."""
    T = shim.DeviceTensor
    nl = len(net.layers)
    hin, hout = {}, {}
    for k, (x, w, dy) in net.host.items():
        px, pw, pdy = (ctx.pinned_empty(a.shape, a.dtype) for a in (x, w, dy))
        px[...], pw[...], pdy[...] = x, w, dy
        hin[k] = (px, pw, pdy)
        hout[k] = (ctx.pinned_empty(dy.shape, DTYPE), ctx.pinned_empty(x.shape, DTYPE), ctx.pinned_empty(w.shape, net.buckets.dtype))
    # device staging in the reference's layout, one set per layer (no reuse hazards inside a step)
    Xn = [T(ctx, net.X[i].shape, DTYPE, "nchw") for i in range(nl)]
    DYn = [T(ctx, net.DY[i].shape, DTYPE, "nchw") for i in range(nl)]
    Yn = [T(ctx, net.Y[i].shape, DTYPE, "nchw") for i in range(nl)]
    DXn = [T(ctx, net.DX[i].shape, DTYPE, "nchw") for i in range(nl)]
    h2d = d2h = 0
    for i in range(nl):
        a, b = hin[net.idx[i]], hout[net.idx[i]]
        h2d += sum(v.nbytes for v in a)
        d2h += sum(v.nbytes for v in b)

    def upload(i):
        px, pw, pdy = hin[net.idx[i]]
        ctx.h2d_bg(Xn[i].ptr, px)
        ctx.h2d_bg(net.W[i].ptr, pw)
        ctx.h2d_bg(DYn[i].ptr, pdy)

    def e2e_step():
        upload(nl - 1)
        for j, i in enumerate(net.order):                     # backward order, so that the buckets fill as in the timed step
            lay = net.layers[i]
            ctx.join_uploads()
            if j + 1 < nl:
                upload(net.order[j + 1])                      # the next layer travels while this one computes
            ctx.nchw_to_nhwc(Xn[i].ptr, net.X[i].ptr, *net.X[i].shape, DTYPE)
            ctx.nchw_to_nhwc(DYn[i].ptr, net.DY[i].ptr, *net.DY[i].shape, DTYPE)
            ctx.prepack([net.descs[i]], [net.W[i].ptr])       # the filters just arrived: pack them for both passes
            net.fwd(i)
            ctx.nhwc_to_nchw(net.Y[i].ptr, Yn[i].ptr, *net.Y[i].shape, DTYPE)
            py, pdx, pdw = hout[net.idx[i]]
            ctx.d2h_bg(py, Yn[i].ptr)
            net.wgrad(i)
            net.dgrad(i)
            ctx.nhwc_to_nchw(net.DX[i].ptr, DXn[i].ptr, *net.DX[i].shape, DTYPE)
            ctx.d2h_bg(pdx, DXn[i].ptr)
            if collective:
                net.buckets.ready(j)
        if collective:
            net.buckets.wait()
        for j, i in enumerate(net.order):
            ctx.d2h_bg(hout[net.idx[i]][2], net.buckets.ptr(j))
        ctx.sync()

    e2e_step()
    e2e_steps = max(2, min(args.steps, 3))
    ts = []
    for _ in range(e2e_steps):
        ctx.barrier()
        t0 = time.perf_counter()
        e2e_step()
        ts.append(time.perf_counter() - t0)
    ts = np.asarray(ts, np.float64)
    if world > 1:
        import torch
        t = torch.from_numpy(ts.copy())
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts = t.numpy()
    e2e_ms = 1e3 * float(ts.mean())
    for t in Xn + DYn + Yn + DXn:
        t.free()
    return {"value": step_flops(BATCH) * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
            "images_per_s": BATCH * world / (e2e_ms * 1e-3),
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
            "path": "per layer: pinned host NCHW x, w, dy -> H2D -> channels-last conversion -> forward, gradWeights, gradInputs -> "
                    "NCHW conversion -> D2H of y, dx, dw; uploads and downloads on background streams beside the kernels; wall clock"}


def run_e2e_theano(net):
    """The same step through the Theano plug-in: for every layer one function compiled by the
    reference's own compiler from T.nnet.conv2d and theano.grad (the optimizer swaps the B200 ops in),
    called with pageable float16 host arrays in the reference's layout; every call copies in (through
    the library's pinned staging buffers and copy threads), runs and copies out (theano/gof/op.py:744-779 is the callback contract).  Wall clock of one pass over
    the 53 layers after a pass over the distinct shapes."""
    try:
        from oracle import ref_theano
        if not ref_theano.available():
            return {"unavailable": "no importable reference here"}
        theano = ref_theano.import_theano()
        import theano_b200.opt  # noqa: F401  (registers the optimizers)
        T = theano.tensor
        fns = {}
        for k, (x, w, dy) in net.host.items():
            lay = WL.RESNET50[k]
            xs, ws, gs = (T.tensor4(dtype="float16") for _ in range(3))
            y = T.nnet.conv2d(xs, ws, border_mode=(lay["p"], lay["p"]), subsample=(lay["s"], lay["s"]), filter_flip=True)
            dw, dx = theano.grad(None, [ws, xs], known_grads={y: gs})
            f = theano.function([xs, ws, gs], [y, dx, dw])
            ops = [type(n.op).__name__ for n in f.maker.fgraph.toposort()]
            assert "B200Conv2d" in ops and "B200Conv2d_gradInputs" in ops and "B200Conv2d_gradWeights" in ops, ops
            fns[k] = f
        for k, f in fns.items():
            f(*net.host[k])
        t0 = time.perf_counter()
        for k in net.idx:
            fns[k](*net.host[k])
        dt = time.perf_counter() - t0
        return {"value": step_flops(net.batch) / dt / 1e12, "unit": "TFLOP/s", "ms_per_step": 1e3 * dt,
                "images_per_s": net.batch / dt,
                "path": "theano.function per layer (T.nnet.conv2d + theano.grad, B200 ops swapped in by the optimizer), pageable "
                        "float16 NCHW host arrays in and out of every call; one pass over the 53 layers, wall clock"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:160])}


def other_configs(ctx, shim, pk):
    """The other benchmark configurations, device-timed (median of 5 per layer and direction, L2
    flushed before each measurement): the single float32 ResNet 3x3 layer and the VGG-16 forward
    stack with fused bias + ReLU."""
    from theano_b200 import layer_bench
    out = {}
    for name, key in (("cfg2", "resnet3x3_f32_N128_C256_K256_14x14_fwd+gradInputs+gradWeights"),
                      ("vgg16", "vgg16_13convs_f32_N64_224x224_fwd+bias+relu")):
        cfg = WL.CONFIGS[name]
        tot_ms = tot_fl = tot_bound = 0.0
        peak = pk["f16"] / 2.0           # kind::tf32 runs at half the 16-bit rate
        for i, lay in enumerate(cfg["layers"]):
            ms, fl, nb, _ = layer_bench.run_layer(ctx, lay, cfg["batch"], cfg["dtype"], cfg["dirs"], cfg["relu"], 5, 1234 + i)
            for t in ms.values():
                tot_ms += t * lay["n"]
                tot_fl += fl * lay["n"]
                tot_bound += max(fl / (peak * 1e12), nb / (pk["hbm"] * 1e9)) * 1e3 * lay["n"]
        out[key] = {"ms": tot_ms, "tflops": tot_fl / tot_ms / 1e9, "frac_of_tf32_peak": tot_fl / tot_ms / 1e9 / peak,
                    "frac_of_summed_rooflines": tot_bound / tot_ms, "images_per_s": cfg["batch"] / (tot_ms * 1e-3),
                    "dtype": "tf32", "timing": "sum over layers of the median of 5 CUDA-event measurements, L2 flushed before each"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="issue every call eagerly (no CUDA graph replay)")
    ap.add_argument("--dw-dtype", default="f32", choices=["f16", "f32"],
                    help="type of the filter-gradient buckets and of their all-reduce")
    ap.add_argument("--bucket-mb", type=int, default=8, help="smallest gradient bucket in MB")
    ap.add_argument("--comm-sms", type=int, default=4,
                    help="with several GPUs: CTAs NCCL may use = SMs the convolution kernels leave free")
    ap.add_argument("--no-autotune", action="store_true",
                    help="no timing-based choice between kernel variants (for runs under a profiler, "
                         "whose replays distort the timings): the static preference order is used")
    ap.add_argument("--no-collective", action="store_true",
                    help="diagnosis only: leave out the all-reduces (the printed line is then not a valid result)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (for runs under a profiler)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-others", action="store_true", help="skip the other configurations' short measurements")
    ap.add_argument("--dump-layers", default=None, help="write the per-layer kernel times of the eager pass to this file (JSON lines)")
    ap.add_argument("--clock-warm", type=int, default=60,
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
