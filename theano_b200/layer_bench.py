"""Per-layer timings of the convolution kernels on the benchmark networks' layer shapes.

    python -m theano_b200.layer_bench --config cfg1|cfg2|vgg16|sweep|resnet50 [--batch N] [--iters K]
                                      [--only I] [--dirs fwd,dgrad,wgrad] [--no-autotune]

`--only I` runs the I-th layer of the configuration alone and `--dirs` a subset of the passes (a
small case for a profiler capture); `--no-autotune` keeps the static choice between kernel
variants (a profiler's replays distort the timings the choice is made from).

Each layer is run in isolation on seeded synthetic tensors kept in HBM in channels-last order
(fresh tensors of the right shape per layer: the networks' names only supply the shapes).
For every direction the time is the median of K CUDA-event measurements on the library's
stream, with the L2 flushed before each one.  VGG-16 layers that are followed by a 2x2 max pooling run it in their epilogue.  Next to it: TFLOP/s from the algorithmic FLOP
count 2*N*K*(C/g)*kH*kW*Ho*Wo, and the fraction of the layer's roofline time
max(FLOP / tensor peak, algorithmic bytes / HBM bandwidth), with bytes = |X| + |W| + |Y|.
One JSON line per layer and one summary line are printed.
"""
import argparse
import json
import os
import sys

import numpy as np

from . import hostlogic, shim
from .workloads import CONFIGS, random_tensor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def run_layer(ctx, lay, batch, dtype, dirs, relu, iters, seed):
    C, K, ks, s, p, H, g, d = lay["C"], lay["K"], lay["k"], lay["s"], lay["p"], lay["H"], lay["g"], lay["d"]
    xshape, wshape = (batch, C, H, H), (K, C // g, ks, ks)
    kw = dict(border_mode=(p, p), subsample=(s, s), filter_dilation=(d, d), num_groups=g, filter_flip=True)
    yshape, _ = hostlogic.forward_shape(xshape, wshape, kw["border_mode"], kw["subsample"], kw["filter_dilation"], g)
    T = shim.DeviceTensor
    X = T.from_host(ctx, random_tensor(seed, xshape, dtype), "nhwc")
    W = T.from_host(ctx, random_tensor(seed + 1, wshape, dtype, np.sqrt(2.0 / ((C // g) * ks * ks))))
    B = T.from_host(ctx, np.zeros((1, K, 1, 1), dtype)) if relu else None
    DY = T.from_host(ctx, random_tensor(seed + 2, yshape, dtype, 0.1 if dtype == np.float16 else 1.0), "nhwc") \
        if ("dgrad" in dirs or "wgrad" in dirs) else None
    pool = bool(lay.get("pool")) and "fwd" in dirs
    Y = T(ctx, (yshape[0], yshape[1], yshape[2] // 2, yshape[3] // 2) if pool else yshape, dtype, "nhwc")
    DX = T(ctx, xshape, dtype, "nhwc") if "dgrad" in dirs else None
    DW = T(ctx, wshape, dtype) if "wgrad" in dirs else None
    calls = {
        "fwd": lambda: shim.device_conv2d(X, W, bias=B, relu=relu, out=Y, pool=pool, **kw),
        "dgrad": lambda: shim.device_grad_inputs(W, DY, (H, H), out=DX, **kw),
        "wgrad": lambda: shim.device_grad_weights(X, DY, (ks, ks), out=DW, **kw),
    }
    es = np.dtype(dtype).itemsize
    flops = hostlogic.conv_flops(xshape, wshape, yshape)
    nbytes = es * (np.prod(xshape) + np.prod(wshape) + np.prod(yshape) / (4.0 if pool else 1.0))
    res = {}
    for name in dirs:
        for _ in range(3):
            calls[name]()
        ts = []
        for _ in range(iters):
            ctx.flush_l2()
            ctx.timer_start()
            calls[name]()
            ts.append(ctx.timer_stop())
        res[name] = float(np.median(ts))
    for t in (X, W, B, DY, Y, DX, DW):
        if t is not None:
            t.free()
    return res, float(flops), float(nbytes), yshape


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="cfg2", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--only", type=int, default=None, help="index of the one layer to run")
    ap.add_argument("--dirs", default=None, help="comma-separated subset of fwd,dgrad,wgrad")
    ap.add_argument("--no-autotune", action="store_true")
    args = ap.parse_args(argv)
    cfg = dict(CONFIGS[args.config])
    if args.only is not None:
        cfg["layers"] = [cfg["layers"][args.only]]
    if args.dirs:
        cfg["dirs"] = tuple(d for d in args.dirs.split(",") if d in cfg["dirs"])
    batch = args.batch or cfg["batch"]
    bf16, hbm, src = peaks()
    peak = bf16 if cfg["dtype"] == np.float16 else bf16 / 2.0
    ctx = shim.Context(args.device)
    if args.no_autotune:
        ctx.set_autotune(False)
    tot_ms, tot_fl, tot_bound = {}, 0.0, {}
    for i, lay in enumerate(cfg["layers"]):
        ms, fl, nb, yshape = run_layer(ctx, lay, batch, cfg["dtype"], cfg["dirs"], cfg["relu"], args.iters, 1234 + i)
        bound_ms = max(fl / (peak * 1e12), nb / (hbm * 1e9)) * 1e3
        kind = "tensor" if fl / (peak * 1e12) >= nb / (hbm * 1e9) else "hbm"
        line = {"layer": "%d->%d %dx%d s%d d%d g%d @%d%s" % (lay["C"], lay["K"], lay["k"], lay["k"], lay["s"], lay["d"], lay["g"], lay["H"],
                                                             " +pool" if lay.get("pool") else ""),
                "count": lay["n"], "batch": batch, "dtype": np.dtype(cfg["dtype"]).name, "gflop": fl / 1e9,
                "bound": kind, "roofline_ms": bound_ms}
        for name, t in ms.items():
            line[name] = {"ms": t, "tflops": fl / t / 1e9, "frac_of_roofline": bound_ms / t}
            tot_ms[name] = tot_ms.get(name, 0.0) + t * lay["n"]
            tot_bound[name] = tot_bound.get(name, 0.0) + bound_ms * lay["n"]
        tot_fl += fl * lay["n"]
        print(json.dumps(line))
        sys.stdout.flush()
    summary = {"config": args.config, "batch": batch, "dtype": np.dtype(cfg["dtype"]).name,
               "gflop_per_pass": tot_fl / 1e9, "peak_tflops": peak, "hbm_gbs": hbm, "peak_source": src}
    all_ms = 0.0
    for name, t in tot_ms.items():
        summary[name] = {"ms": t, "tflops": tot_fl / t / 1e9, "frac_of_peak": tot_fl / t / 1e9 / peak,
                         "frac_of_roofline": tot_bound[name] / t}
        all_ms += t
    summary["images_per_s"] = batch / (all_ms * 1e-3)
    print(json.dumps(summary))


if __name__ == "__main__":
    main()
